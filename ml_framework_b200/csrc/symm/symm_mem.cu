// Symmetric (peer-mapped) memory and the collectives that run over it.
//
// Every rank allocates buffers of identical size, exports them as CUDA IPC handles, and maps
// every peer's buffer into its own address space, so a kernel can load from / store to any
// rank's copy directly over NVLink (through NVSwitch every peer is one hop away). On top of
// that this file provides:
//   * a device-side barrier over a signal pad (bounded wait, error status instead of a hang),
//   * reduce-scatter of gradient buckets by direct peer reads with unscale and overflow
//     detection fused (each rank sums its slice of all W copies in fp32),
//   * two-shot all-reduce for DDP buckets (reduce own slice, then store it to every peer),
//   * one-shot all-reduce for small latency-bound messages (tensor-parallel decode).
// Kernels that wait on peers are separate launches from kernels that move data, so the data
// kernels can be validated on one GPU with every "rank" buffer local.
//
// Reference semantics: ring reduce-scatter / all-gather
// (src/MLFramework/Distributed/RingAllReduce.cs:86-163, FSDP/ReduceScatterOperation.cs:54-125),
// bucket all-reduce (src/MLFramework/Distributed/GradientBucket.cs:112-126), algorithm choice by
// message size (src/MLFramework/Communication/Optimizations/AlgorithmSelector.cs:24-65). On
// NVSwitch ring / tree schedules bring nothing: small messages go one-shot, large ones two-shot.
#include <float.h>

#include "../common/host.h"
#include "../common/ptx.cuh"
#include "../mlf_api.h"

namespace mlf {

struct PeerPtrs {
  void* p[8];
};

// ------------------------------------------------------------------------------------------
// barrier: pad[r] is rank r's signal pad (uint32 [8 x 32] : slot s*32 written by rank s).
// ------------------------------------------------------------------------------------------
__global__ void symm_barrier_kernel(PeerPtrs pads, int rank, int world, uint32_t epoch, int* err) {
  const int t = threadIdx.x;
  if (t < world) {
    uint32_t* remote = static_cast<uint32_t*>(pads.p[t]) + rank * 32;
    __threadfence_system();
    st_release_sys(remote, epoch);
  }
  if (t < world) {
    const uint32_t* mine = static_cast<const uint32_t*>(pads.p[rank]) + t * 32;
    wait_flag_ge_sys(mine, epoch, err, ERR_WAIT_PEER_FLAG);
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------
// segment table: the same layout on every rank
// ------------------------------------------------------------------------------------------
struct ReduceSeg {
  long long src_off;   // element offset of this rank's slice inside every rank's full buffer
  long long dst_off;   // element offset in the local output
  long long numel;     // elements in the slice
};

// out[dst_off + i] = scale * sum_r bufs[r][src_off + i]   (bf16 in, bf16 or fp32 out)
// found_inf is raised when a reduced value is not finite; sumsq accumulates the squared norm.
// Sum of the same 16-byte vector of all W buffers, for U vectors per thread at once: every peer load is issued
// before the first use, so a thread keeps U * W loads of 16 bytes in flight over NVLink (the reductions are
// bound by bytes in flight, not by arithmetic). MAXW bounds the unrolled rank loop.
template <int U, int MAXW>
__device__ __forceinline__ void peer_sum(const PeerPtrs& bufs, int world, int rank, long long elem_base, long long i0, long long stride,
                                         long long nvec, float (&a)[U][8]) {
  uint4 v[U][MAXW];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const long long i = i0 + u * stride;
#pragma unroll
    for (int k = 0; k < MAXW; ++k) {
      if (k < world && i < nvec) {
        int r = rank + 1 + k;       // start with the next rank so the links are used evenly
        if (r >= world) r -= world;
        v[u][k] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(bufs.p[r]) + elem_base + i * 8);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
#pragma unroll
    for (int j = 0; j < 8; ++j) a[u][j] = 0.f;
    const long long i = i0 + u * stride;
#pragma unroll
    for (int k = 0; k < MAXW; ++k) {
      if (k < world && i < nvec) {
        float2 f0 = unpack_bf16x2(v[u][k].x), f1 = unpack_bf16x2(v[u][k].y), f2 = unpack_bf16x2(v[u][k].z), f3 = unpack_bf16x2(v[u][k].w);
        a[u][0] += f0.x; a[u][1] += f0.y; a[u][2] += f1.x; a[u][3] += f1.y; a[u][4] += f2.x; a[u][5] += f2.y; a[u][6] += f3.x; a[u][7] += f3.y;
      }
    }
  }
}

template <typename OutT, int U, int MAXW>
__device__ __forceinline__ void rs_reduce_span(const PeerPtrs& bufs, int world, int rank, const ReduceSeg* segs, int n_segs, OutT* out,
                                               float sc, bool& bad, float& acc_sq) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int s = 0; s < n_segs; ++s) {
    const ReduceSeg sg = segs[s];
    const long long nvec = sg.numel / 8;
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
      float a[U][8];
      peer_sum<U, MAXW>(bufs, world, rank, sg.src_off, i0, stride, nvec, a);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i >= nvec) break;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          a[u][j] *= sc;
          if (!isfinite(a[u][j])) bad = true;
          acc_sq += a[u][j] * a[u][j];
        }
        OutT* o = out + sg.dst_off + i * 8;
        if (sizeof(OutT) == 2) {
          uint4 w;
          w.x = pack_bf16x2(a[u][0], a[u][1]); w.y = pack_bf16x2(a[u][2], a[u][3]); w.z = pack_bf16x2(a[u][4], a[u][5]); w.w = pack_bf16x2(a[u][6], a[u][7]);
          *reinterpret_cast<uint4*>(o) = w;
        } else {
          reinterpret_cast<float4*>(o)[0] = make_float4(a[u][0], a[u][1], a[u][2], a[u][3]);
          reinterpret_cast<float4*>(o)[1] = make_float4(a[u][4], a[u][5], a[u][6], a[u][7]);
        }
      }
    }
  }
}

template <typename OutT>
__device__ __forceinline__ void rs_reduce_body(const PeerPtrs& bufs, int world, int rank, const ReduceSeg* segs, int n_segs, OutT* out,
                                               float sc, bool& bad, float& acc_sq) {
  if (world <= 2) rs_reduce_span<OutT, 4, 2>(bufs, world, rank, segs, n_segs, out, sc, bad, acc_sq);
  else if (world <= 4) rs_reduce_span<OutT, 2, 4>(bufs, world, rank, segs, n_segs, out, sc, bad, acc_sq);
  else rs_reduce_span<OutT, 2, 8>(bufs, world, rank, segs, n_segs, out, sc, bad, acc_sq);
}

template <typename OutT>
__global__ void __launch_bounds__(256)
rs_reduce_kernel(PeerPtrs bufs, int world, int rank, const ReduceSeg* segs, int n_segs, OutT* out, float scale,
                 const float* scale_ptr, int* found_inf, float* sumsq) {
  const float sc = scale * (scale_ptr ? *scale_ptr : 1.f);
  float acc_sq = 0.f;
  bool bad = false;
  rs_reduce_body<OutT>(bufs, world, rank, segs, n_segs, out, sc, bad, acc_sq);
  if (found_inf && __any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(found_inf, 1);
  if (sumsq) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc_sq += __shfl_xor_sync(0xffffffffu, acc_sq, o);
    if ((threadIdx.x & 31) == 0 && isfinite(acc_sq)) atomicAdd(sumsq, acc_sq);
  }
}

// Two-shot all-reduce, in place over symmetric buffers: rank r reduces slice r of all copies and
// stores the result into slice r of every rank's buffer. A barrier must separate it from the
// producers before and from the consumers after.
__global__ void __launch_bounds__(256)
ar_two_shot_kernel(PeerPtrs bufs, int world, int rank, long long numel, float scale) {
  const long long per = ((numel / 8 + world - 1) / world) * 8;
  const long long lo = per * rank;
  const long long hi = lo + per < numel ? lo + per : numel;
  const long long nvec = hi > lo ? (hi - lo) / 8 : 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < world) {
        int r = rank + 1 + k;
        if (r >= world) r -= world;
        v[k] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(bufs.p[r]) + lo + i * 8);
      }
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < world) {
        float2 f0 = unpack_bf16x2(v[k].x), f1 = unpack_bf16x2(v[k].y), f2 = unpack_bf16x2(v[k].z), f3 = unpack_bf16x2(v[k].w);
        a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
      }
    uint4 w;
    w.x = pack_bf16x2(a[0] * scale, a[1] * scale); w.y = pack_bf16x2(a[2] * scale, a[3] * scale);
    w.z = pack_bf16x2(a[4] * scale, a[5] * scale); w.w = pack_bf16x2(a[6] * scale, a[7] * scale);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < world) {
        int r = rank + 1 + k;
        if (r >= world) r -= world;
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(bufs.p[r]) + lo + i * 8) = w;
      }
  }
}

// One-shot all-reduce for small messages: every rank reads all W copies and writes its own
// private output (no second exchange). in: symmetric staging buffers; out: local tensor.
__global__ void __launch_bounds__(256)
ar_one_shot_kernel(PeerPtrs bufs, int world, int rank, __nv_bfloat16* out, long long numel, const __nv_bfloat16* residual) {
  const long long nvec = numel / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < world) v[k] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(bufs.p[k]) + i * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < world) {
        float2 f0 = unpack_bf16x2(v[k].x), f1 = unpack_bf16x2(v[k].y), f2 = unpack_bf16x2(v[k].z), f3 = unpack_bf16x2(v[k].w);
        a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
      }
    if (residual) {
      const uint4 rr = *reinterpret_cast<const uint4*>(residual + i * 8);
      float2 f0 = unpack_bf16x2(rr.x), f1 = unpack_bf16x2(rr.y), f2 = unpack_bf16x2(rr.z), f3 = unpack_bf16x2(rr.w);
      a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
    }
    uint4 w;
    w.x = pack_bf16x2(a[0], a[1]); w.y = pack_bf16x2(a[2], a[3]); w.z = pack_bf16x2(a[4], a[5]); w.w = pack_bf16x2(a[6], a[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = w;
  }
}

// ------------------------------------------------------------------------------------------
// Synchronisation whose epoch lives in device memory, so that a captured CUDA graph replays it:
// pads as above (one signal slot per peer), plus a local {epoch, finished-CTA count} pair. Every
// CTA reads the epoch of this launch (previous + 1); CTA 0 signals the peers; everybody waits for
// all peers' signals; the last CTA to finish publishes the new epoch. All ranks must run the same
// sequence of such launches.
// ------------------------------------------------------------------------------------------
struct SyncState {
  uint32_t epoch;
  uint32_t done;
};

__device__ __forceinline__ uint32_t sync_enter(const PeerPtrs& pads, SyncState* st, int rank, int world, int* err) {
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(&st->epoch) + 1u;
  __syncthreads();
  const uint32_t e = s_epoch;
  const int t = threadIdx.x;
  if (blockIdx.x == 0 && t < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(pads.p[t]) + rank * 32, e);
  }
  if (t < world) wait_flag_ge_sys(static_cast<const uint32_t*>(pads.p[rank]) + t * 32, e, err, ERR_WAIT_PEER_FLAG);
  __syncthreads();
  return e;
}

__device__ __forceinline__ void sync_leave(SyncState* st, uint32_t e) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&st->done, 1u) == gridDim.x - 1) {
      st->done = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(&st->epoch) = e;
    }
  }
}

// Leave with a handshake: the last CTA of this rank to finish tells every peer that all of this
// rank's loads from and stores to peer memory for this launch are complete (epoch e + 1) and waits
// for the same news from every peer, so that when the kernel ends on a rank (a) every peer has
// finished reading this rank's buffers and (b) everything the peers stored here is visible. The
// device epoch advances by two per launch.
__device__ __forceinline__ void sync_leave_all(const PeerPtrs& pads, SyncState* st, int rank, int world, uint32_t e, int* err) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(&st->done, 1u) == gridDim.x - 1 ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(pads.p[t]) + rank * 32, e + 1u);
    wait_flag_ge_sys(static_cast<const uint32_t*>(pads.p[rank]) + t * 32, e + 1u, err, ERR_WAIT_PEER_FLAG);
  }
  __syncthreads();
  if (t == 0) {
    st->done = 0;
    __threadfence();
    *reinterpret_cast<volatile uint32_t*>(&st->epoch) = e + 1u;
  }
}

// Raises the overflow flag of EVERY rank (flags.p[r] = rank r's flag in symmetric memory), so that
// all ranks skip the optimizer step together without a further collective.
__device__ __forceinline__ void raise_flag_everywhere(const PeerPtrs& flags, int world, bool bad) {
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) {
    for (int r = 0; r < world; ++r)
      if (flags.p[r]) *reinterpret_cast<volatile int*>(flags.p[r]) = 1;
  }
}

// Reduce-scatter with both synchronisations inside (replaces barrier + rs_reduce + flag all-reduce):
// waits until every rank has queued the same launch (their producers, earlier on their streams, are
// then complete), sums this rank's slices out of all W buffers, raises every rank's overflow flag on
// a non-finite result, and leaves with the handshake above.
template <typename OutT>
__global__ void __launch_bounds__(256)
rs_reduce_sync_kernel(PeerPtrs bufs, PeerPtrs pads, SyncState* st, PeerPtrs flags, int world, int rank, const ReduceSeg* segs, int n_segs,
                      OutT* out, float scale, const float* scale_ptr, float* sumsq, int* err) {
  const uint32_t e = sync_enter(pads, st, rank, world, err);
  const float sc = scale * (scale_ptr ? *scale_ptr : 1.f);
  float acc_sq = 0.f;
  bool bad = false;
  rs_reduce_body<OutT>(bufs, world, rank, segs, n_segs, out, sc, bad, acc_sq);
  raise_flag_everywhere(flags, world, bad);
  if (sumsq) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc_sq += __shfl_xor_sync(0xffffffffu, acc_sq, o);
    if ((threadIdx.x & 31) == 0 && isfinite(acc_sq)) atomicAdd(sumsq, acc_sq);
  }
  sync_leave_all(pads, st, rank, world, e, err);
}

template <int U, int MAXW>
__device__ __forceinline__ void two_shot_span(const PeerPtrs& bufs, int world, int rank, long long lo, long long nvec, float sc, bool& bad) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    float a[U][8];
    peer_sum<U, MAXW>(bufs, world, rank, lo, i0, stride, nvec, a);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) break;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[u][j] *= sc;
        if (!isfinite(a[u][j])) bad = true;
      }
      uint4 w;
      w.x = pack_bf16x2(a[u][0], a[u][1]); w.y = pack_bf16x2(a[u][2], a[u][3]); w.z = pack_bf16x2(a[u][4], a[u][5]); w.w = pack_bf16x2(a[u][6], a[u][7]);
#pragma unroll
      for (int k = 0; k < MAXW; ++k)
        if (k < world) {
          int r = rank + 1 + k;
          if (r >= world) r -= world;
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(bufs.p[r]) + lo + i * 8) = w;
        }
    }
  }
}

// Two-shot all-reduce of a gradient bucket with both synchronisations inside: rank r sums slice r of
// all W copies, scales it, checks it for overflow (raising every rank's flag) and stores it into
// slice r of every rank's buffer. When the kernel ends on a rank its whole buffer holds the result.
__global__ void __launch_bounds__(256)
ar_two_shot_sync_kernel(PeerPtrs bufs, PeerPtrs pads, SyncState* st, PeerPtrs flags, int world, int rank, long long numel, float scale,
                        const float* scale_ptr, int* err) {
  const uint32_t e = sync_enter(pads, st, rank, world, err);
  const float sc = scale * (scale_ptr ? *scale_ptr : 1.f);
  const long long per = ((numel / 8 + world - 1) / world) * 8;
  const long long lo = per * rank;
  const long long hi = lo + per < numel ? lo + per : numel;
  const long long nvec = hi > lo ? (hi - lo) / 8 : 0;
  bool bad = false;
  if (world <= 2) two_shot_span<4, 2>(bufs, world, rank, lo, nvec, sc, bad);
  else if (world <= 4) two_shot_span<2, 4>(bufs, world, rank, lo, nvec, sc, bad);
  else two_shot_span<2, 8>(bufs, world, rank, lo, nvec, sc, bad);
  raise_flag_everywhere(flags, world, bad);
  sync_leave_all(pads, st, rank, world, e, err);
}

// One-shot all-reduce with the arrival synchronisation inside: the producers of bufs[*] (the kernels
// before this one on every rank's stream) are complete once all peers have signalled.
__global__ void __launch_bounds__(256)
ar_one_shot_sync_kernel(PeerPtrs bufs, PeerPtrs pads, SyncState* st, int world, int rank, __nv_bfloat16* out, long long numel,
                        const __nv_bfloat16* residual, int* err) {
  const uint32_t e = sync_enter(pads, st, rank, world, err);
  const long long nvec = numel / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < world) v[k] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(bufs.p[k]) + i * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < world) {
        float2 f0 = unpack_bf16x2(v[k].x), f1 = unpack_bf16x2(v[k].y), f2 = unpack_bf16x2(v[k].z), f3 = unpack_bf16x2(v[k].w);
        a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
      }
    if (residual) {
      const uint4 rr = *reinterpret_cast<const uint4*>(residual + i * 8);
      float2 f0 = unpack_bf16x2(rr.x), f1 = unpack_bf16x2(rr.y), f2 = unpack_bf16x2(rr.z), f3 = unpack_bf16x2(rr.w);
      a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
    }
    uint4 w;
    w.x = pack_bf16x2(a[0], a[1]); w.y = pack_bf16x2(a[2], a[3]); w.z = pack_bf16x2(a[4], a[5]); w.w = pack_bf16x2(a[6], a[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = w;
  }
  sync_leave(st, e);
}

// Greedy sampling over a vocabulary split across ranks. Step 1 (every rank): best (value, global index)
// of each row of the local logits into this rank's staging buffer. Step 2: synchronise, read all
// ranks' candidates, keep the best (lowest index on ties).
struct ArgmaxCand {
  float value;
  int index;
};

__global__ void __launch_bounds__(256)
argmax_local_kernel(const __nv_bfloat16* logits, long long ld, int cols, int index_base, int vocab, ArgmaxCand* cand) {
  const long long r = blockIdx.x;
  const __nv_bfloat16* row = logits + r * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < cols && index_base + i < vocab; i += blockDim.x) {
    const float v = __bfloat162float(row[i]);
    if (v > best) { best = v; bi = index_base + i; }
  }
  __shared__ float sv[256];
  __shared__ int si[256];
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float ov = sv[threadIdx.x + s];
      const int oi = si[threadIdx.x + s];
      if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) { sv[threadIdx.x] = ov; si[threadIdx.x] = oi; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) { cand[r].value = sv[0]; cand[r].index = si[0]; }
}

__global__ void __launch_bounds__(256)
argmax_combine_sync_kernel(PeerPtrs bufs, PeerPtrs pads, SyncState* st, int world, int rank, long long rows, long long* out, int* err) {
  const uint32_t e = sync_enter(pads, st, rank, world, err);
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (long long)gridDim.x * blockDim.x) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int k = 0; k < world; ++k) {
      const ArgmaxCand c = static_cast<const ArgmaxCand*>(bufs.p[k])[r];
      if (c.value > best || (c.value == best && c.index < bi)) { best = c.value; bi = c.index; }
    }
    out[r] = bi == 0x7fffffff ? 0 : bi;
  }
  sync_leave(st, e);
}

// ------------------------------------------------------------------------------------------
// Cross-entropy over a vocabulary split across ranks (tensor-parallel LM head). Each rank holds the
// logits of its own vocabulary columns [T, Vl] (global columns lo .. lo + Vl). Step 1 reduces every
// row to three numbers (local maximum, sum of exponentials against it, the target's logit when the
// target is one of this rank's columns) in this rank's statistics buffer; step 2 combines the W
// statistics of a row, writes the row's loss and overwrites the local logits with
// d loss / d logits * gscale. With do_sync the statistics buffers are peer-mapped and step 2 waits
// inside the kernel until every rank has finished step 1; otherwise stats.p[r] are local copies
// (after a process-group all-gather, or W = 1).
// ------------------------------------------------------------------------------------------
struct VpStat {
  float mx, se, tl, pad;
};

__global__ void __launch_bounds__(256)
vp_ce_stats_kernel(const __nv_bfloat16* logits, long long ld, const long long* targets, int T, int valid_cols, long long lo,
                   VpStat* stats, int* err) {
  __shared__ float red_a[8], red_b[8];
  const int nvec = valid_cols / 8;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const __nv_bfloat16* row = logits + (long long)t * ld;
    float mx = -FLT_MAX, se = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 u = reinterpret_cast<const uint4*>(row)[i];
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
    for (int i = nvec * 8 + threadIdx.x; i < valid_cols; i += blockDim.x) {
      const float f = __bfloat162float(row[i]);
      if (f > mx) { se *= __expf(mx - f); mx = f; }
      se += __expf(f - mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, mx, o), os = __shfl_xor_sync(0xffffffffu, se, o);
      const float nm = fmaxf(mx, om);
      se = se * __expf(mx - nm) + os * __expf(om - nm);
      mx = nm;
    }
    const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();      // red_* of the previous row are consumed
    if ((threadIdx.x & 31) == 0) { red_a[w] = mx; red_b[w] = se; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float gm = red_a[0], gsum = red_b[0];
      for (int k = 1; k < nw; ++k) {
        const float nm = fmaxf(gm, red_a[k]);
        gsum = gsum * __expf(gm - nm) + red_b[k] * __expf(red_a[k] - nm);
        gm = nm;
      }
      const long long tg = targets[t] - lo;
      VpStat st;
      st.mx = gm; st.se = gsum; st.pad = 0.f;
      st.tl = (targets[t] >= 0 && tg >= 0 && tg < valid_cols) ? __bfloat162float(row[tg]) : 0.f;
      *reinterpret_cast<float4*>(stats + t) = *reinterpret_cast<float4*>(&st);
    }
  }
}

__global__ void __launch_bounds__(256)
vp_ce_grad_kernel(__nv_bfloat16* logits, long long ld, int Vl, const long long* targets, int T, int valid_cols, long long lo, long long vocab,
                  PeerPtrs stats, PeerPtrs pads, SyncState* st, int world, int rank, int do_sync, float* loss_rows, float* loss_sum,
                  float gscale, const float* gscale_ptr, float loss_weight, int* err) {
  uint32_t e = 0;
  if (do_sync) e = sync_enter(pads, st, rank, world, err);
  __shared__ float s_gm, s_inv, s_ignore;
  const float gs = gscale * (gscale_ptr ? *gscale_ptr : 1.f);
  const int nvec = Vl / 8;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const long long tgt = targets[t];
    if (threadIdx.x == 0) {
      float gm = -FLT_MAX, gsum = 0.f, tl = 0.f;
      for (int r = 0; r < world; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(static_cast<const VpStat*>(stats.p[r]) + t);
        const float nm = fmaxf(gm, v.x);
        gsum = gsum * __expf(gm - nm) + v.y * __expf(v.x - nm);
        gm = nm;
        tl += v.z;
      }
      const bool ignore = tgt < 0;
      if (!ignore && tgt >= vocab) atomicCAS(err, 0, ERR_BAD_INDEX);
      const float l = (ignore || tgt >= vocab) ? 0.f : gm + __logf(gsum) - tl;
      if (loss_rows) loss_rows[t] = l;
      if (loss_sum) atomicAdd(loss_sum, l * loss_weight);
      s_gm = gm; s_inv = 1.f / gsum; s_ignore = ignore ? 1.f : 0.f;
    }
    __syncthreads();
    const float gm = s_gm, inv = s_inv;
    const bool ignore = s_ignore != 0.f;
    const long long tl_col = tgt - lo;
    __nv_bfloat16* row = logits + (long long)t * ld;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const uint4 u = reinterpret_cast<const uint4*>(row)[i];
      float f[8];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = i * 8 + j;
        float g = (ignore || col >= valid_cols) ? 0.f : __expf(f[j] - gm) * inv;
        if (!ignore && (long long)col == tl_col) g -= 1.f;
        f[j] = g * gs;
      }
      uint4 o;
      o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]); o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
      reinterpret_cast<uint4*>(row)[i] = o;
    }
    for (int col = nvec * 8 + threadIdx.x; col < Vl; col += blockDim.x) {
      float g = (ignore || col >= valid_cols) ? 0.f : __expf(__bfloat162float(row[col]) - gm) * inv;
      if (!ignore && (long long)col == tl_col) g -= 1.f;
      row[col] = __float2bfloat16(g * gs);
    }
    __syncthreads();      // s_* are rewritten for the next row
  }
  if (do_sync) sync_leave_all(pads, st, rank, world, e, err);
}

// out[row, :] = sum_w partial[w, row, :] (+ bias) (+ residual): the second half of GEMM->reduce-
// scatter, where peers have stored their partial tiles into this rank's [W, rows, cols] buffer.
__global__ void __launch_bounds__(256)
sum_partials_kernel(const __nv_bfloat16* partial, int world, long long rows, int cols, __nv_bfloat16* out, long long ldo,
                    const __nv_bfloat16* bias, const __nv_bfloat16* residual, long long ldr) {
  const int vpr = cols / 8;
  const long long total = rows * vpr;
  const long long plane = rows * (long long)cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int c = (int)(i % vpr) * 8;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int w = 0; w < world; ++w) {
      const uint4 v = *reinterpret_cast<const uint4*>(partial + w * plane + r * cols + c);
      float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
      a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
    }
    if (bias) {
      const uint4 v = *reinterpret_cast<const uint4*>(bias + c);
      float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
      a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
    }
    if (residual) {
      const uint4 v = *reinterpret_cast<const uint4*>(residual + r * ldr + c);
      float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
      a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
    }
    uint4 w;
    w.x = pack_bf16x2(a[0], a[1]); w.y = pack_bf16x2(a[2], a[3]); w.z = pack_bf16x2(a[4], a[5]); w.w = pack_bf16x2(a[6], a[7]);
    *reinterpret_cast<uint4*>(out + r * ldo + c) = w;
  }
}

// The same sum with the arrival synchronisation inside: every rank has queued this launch, so its GEMM (earlier on its
// stream) has finished storing partial tiles into the peers' buffers. Nothing waits at the end; callers alternate
// between two partial buffers, and the arrival wait of call n + 1 is what tells a rank that every peer has finished
// the sum of call n - 1 before new tiles are stored over it.
__global__ void __launch_bounds__(256)
sum_partials_sync_kernel(PeerPtrs pads, SyncState* st, int world, int rank, const __nv_bfloat16* partial, long long rows, int cols,
                         __nv_bfloat16* out, long long ldo, const __nv_bfloat16* bias, const __nv_bfloat16* residual, long long ldr,
                         int* err) {
  const uint32_t e = sync_enter(pads, st, rank, world, err);
  const int vpr = cols / 8;
  const long long total = rows * vpr;
  const long long plane = rows * (long long)cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int c = (int)(i % vpr) * 8;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    auto add8 = [&](const uint4 v) {
      float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
      a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y; a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
    };
    uint4 v[8];
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < world) v[w] = *reinterpret_cast<const uint4*>(partial + w * plane + r * cols + c);      // all W loads in flight before the first add
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < world) add8(v[w]);
    if (bias) add8(*reinterpret_cast<const uint4*>(bias + c));
    if (residual) add8(*reinterpret_cast<const uint4*>(residual + r * ldr + c));
    uint4 w;
    w.x = pack_bf16x2(a[0], a[1]); w.y = pack_bf16x2(a[2], a[3]); w.z = pack_bf16x2(a[4], a[5]); w.w = pack_bf16x2(a[6], a[7]);
    *reinterpret_cast<uint4*>(out + r * ldo + c) = w;
  }
  sync_leave(st, e);
}

// Plain multi-segment copy from peers (all-gather without a GEMM attached).
struct CopySegHost {
  const void* src;
  void* dst;
  long long bytes;
};
__global__ void __launch_bounds__(512) peer_copy_kernel(const CopySegHost* segs, int n_segs) {
  for (int s = 0; s < n_segs; ++s) {
    const CopySegHost sg = segs[s];
    const uint4* src = static_cast<const uint4*>(sg.src);
    uint4* dst = static_cast<uint4*>(sg.dst);
    const long long n = sg.bytes / 16;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long step = (long long)gridDim.x * blockDim.x;
    // eight 16-byte loads in flight per thread: a copy over NVLink is bound by bytes in flight
    for (; i + 7 * step < n; i += 8 * step) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = src[i + k * step];
#pragma unroll
      for (int k = 0; k < 8; ++k) dst[i + k * step] = v[k];
    }
    for (; i < n; i += step) dst[i] = src[i];
  }
}

}  // namespace mlf

using namespace mlf;

// ---- allocation and IPC --------------------------------------------------------------------
MLF_API int mlf_symm_alloc(long long bytes, void** ptr, unsigned char* handle64) {
  MLF_REQUIRE(bytes > 0 && ptr && handle64, "symm_alloc: bad arguments");
  void* p = nullptr;
  MLF_CHECK_CUDA(cudaMalloc(&p, (size_t)bytes));
  MLF_CHECK_CUDA(cudaMemset(p, 0, (size_t)bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return check_cuda(e, "cudaIpcGetMemHandle");
  }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return 0;
}
MLF_API int mlf_symm_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  MLF_CHECK_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
MLF_API int mlf_symm_close(void* ptr) {
  MLF_CHECK_CUDA(cudaIpcCloseMemHandle(ptr));
  return 0;
}
MLF_API int mlf_symm_free(void* ptr) {
  MLF_CHECK_CUDA(cudaFree(ptr));
  return 0;
}

static PeerPtrs to_peers(void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < 8; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}

// ---- collectives ---------------------------------------------------------------------------
MLF_API int mlf_symm_barrier(void* const* pads, int rank, int world, unsigned int epoch, uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world, "symm_barrier: bad rank/world");
  symm_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(to_peers(pads, world), rank, world, epoch,
                                                                            device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// segs: device array of {src_off, dst_off, numel} (elements; multiples of 8). out_fp32 selects
// the output type. scale_ptr / found_inf / sumsq are optional device pointers.
MLF_API int mlf_rs_reduce(void* const* bufs, int world, int rank, const void* segs, int n_segs, void* out, int out_fp32,
                          float scale, const float* scale_ptr, int* found_inf, float* sumsq, long long total_numel,
                          uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8, "rs_reduce: world must be 1..8");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  long long g = (total_numel / 8 + 255) / 256;
  const long long cap = (long long)sm_count() * 4;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  if (out_fp32)
    rs_reduce_kernel<float><<<(int)g, 256, 0, st>>>(to_peers(bufs, world), world, rank, static_cast<const ReduceSeg*>(segs),
                                                    n_segs, static_cast<float*>(out), scale, scale_ptr, found_inf, sumsq);
  else
    rs_reduce_kernel<__nv_bfloat16><<<(int)g, 256, 0, st>>>(to_peers(bufs, world), world, rank,
                                                            static_cast<const ReduceSeg*>(segs), n_segs,
                                                            static_cast<__nv_bfloat16*>(out), scale, scale_ptr, found_inf, sumsq);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_ar_two_shot(void* const* bufs, int world, int rank, long long numel, float scale, uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8 && numel % 8 == 0, "ar_two_shot: numel must be a multiple of 8");
  long long g = (numel / 8 / world + 255) / 256;
  const long long cap = (long long)sm_count() * 4;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  ar_two_shot_kernel<<<(int)g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(to_peers(bufs, world), world, rank, numel, scale);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Reduce-scatter / two-shot all-reduce that synchronise inside the kernel (see the kernels above).
// pads / state as for mlf_ar_one_shot_sync; every stream that issues such launches needs a pad and a
// state of its own, and all ranks must issue the same sequence per pad. flags: every rank's overflow
// flag (int, in symmetric memory) or null. max_ctas bounds the grid (0 = one CTA per two SMs), so a
// launch that overlaps compute kernels leaves them most of the SMs.
MLF_API int mlf_rs_reduce_sync(void* const* bufs, void* const* pads, void* state, void* const* flags, int world, int rank,
                               const void* segs, int n_segs, void* out, int out_fp32, float scale, const float* scale_ptr, float* sumsq,
                               long long total_numel, int max_ctas, uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8 && state != nullptr, "rs_reduce_sync: bad arguments");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  long long g = (total_numel / 8 + 255) / 256;
  const long long cap = max_ctas > 0 ? max_ctas : sm_count() / 2;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  PeerPtrs fl = flags ? to_peers(flags, world) : PeerPtrs{};
  if (out_fp32)
    rs_reduce_sync_kernel<float><<<(int)g, 256, 0, st>>>(to_peers(bufs, world), to_peers(pads, world), static_cast<SyncState*>(state), fl,
                                                         world, rank, static_cast<const ReduceSeg*>(segs), n_segs, static_cast<float*>(out),
                                                         scale, scale_ptr, sumsq, device_status_word());
  else
    rs_reduce_sync_kernel<__nv_bfloat16><<<(int)g, 256, 0, st>>>(to_peers(bufs, world), to_peers(pads, world),
                                                                 static_cast<SyncState*>(state), fl, world, rank,
                                                                 static_cast<const ReduceSeg*>(segs), n_segs,
                                                                 static_cast<__nv_bfloat16*>(out), scale, scale_ptr, sumsq,
                                                                 device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_ar_two_shot_sync(void* const* bufs, void* const* pads, void* state, void* const* flags, int world, int rank,
                                 long long numel, float scale, const float* scale_ptr, int max_ctas, uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8 && numel % 8 == 0 && state != nullptr, "ar_two_shot_sync: bad arguments");
  long long g = (numel / 8 / world + 255) / 256;
  const long long cap = max_ctas > 0 ? max_ctas : sm_count() / 2;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  PeerPtrs fl = flags ? to_peers(flags, world) : PeerPtrs{};
  ar_two_shot_sync_kernel<<<(int)g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      to_peers(bufs, world), to_peers(pads, world), static_cast<SyncState*>(state), fl, world, rank, numel, scale, scale_ptr,
      device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_ar_one_shot(void* const* bufs, int world, int rank, void* out, long long numel, const void* residual,
                            uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8 && numel % 8 == 0, "ar_one_shot: numel must be a multiple of 8");
  long long g = (numel / 8 + 255) / 256;
  const long long cap = (long long)sm_count() * 2;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  ar_one_shot_kernel<<<(int)g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      to_peers(bufs, world), world, rank, static_cast<__nv_bfloat16*>(out), numel, static_cast<const __nv_bfloat16*>(residual));
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// One-shot all-reduce that synchronises inside the kernel (no host-side epoch: replayable from a CUDA
// graph). pads: every rank's signal pad (1 KB of slots); state: this rank's 8-byte {epoch, count} pair,
// zero-initialised. Callers alternate between two staging buffers from one call to the next.
MLF_API int mlf_ar_one_shot_sync(void* const* bufs, void* const* pads, void* state, int world, int rank, void* out, long long numel,
                                 const void* residual, uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8 && numel % 8 == 0 && state != nullptr, "ar_one_shot_sync: bad arguments");
  long long g = (numel / 8 + 255) / 256;
  const long long cap = (long long)sm_count();
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  ar_one_shot_sync_kernel<<<(int)g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      to_peers(bufs, world), to_peers(pads, world), static_cast<SyncState*>(state), world, rank, static_cast<__nv_bfloat16*>(out), numel,
      static_cast<const __nv_bfloat16*>(residual), device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Arg-max over a vocabulary split across ranks: logits [rows, cols] are this rank's columns
// [index_base, index_base + cols) of the vocabulary; bufs[r] holds rank r's candidates (8 bytes per row).
MLF_API int mlf_tp_argmax(const void* logits, long long rows, long long ld, int cols, int index_base, int vocab, void* const* bufs,
                          void* const* pads, void* state, int world, int rank, long long* out, uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8 && rows > 0 && state != nullptr, "tp_argmax: bad arguments");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  argmax_local_kernel<<<(int)rows, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, cols, index_base, vocab,
                                                 static_cast<ArgmaxCand*>(bufs[rank]));
  count_launch();
  argmax_combine_sync_kernel<<<1, 256, 0, st>>>(to_peers(bufs, world), to_peers(pads, world), static_cast<SyncState*>(state), world, rank,
                                                rows, out, device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Vocabulary-parallel cross-entropy (see the kernels above). logits [T, ld] bf16 hold this rank's Vl columns of the
// vocabulary starting at global column lo; they are overwritten with the gradient. stats[r]: rank r's statistics
// buffer (16 bytes per row); with do_sync != 0 these are peer-mapped and pads / state are a signal pad and its device
// epoch. loss_sum must be zeroed by the caller.
MLF_API int mlf_vp_cross_entropy(void* logits, long long ld, int Vl, const long long* targets, int T, long long lo, long long vocab,
                                 void* const* stats, void* const* pads, void* state, int world, int rank, int do_sync, float* loss_rows,
                                 float* loss_sum, float gscale, const float* gscale_ptr, float loss_weight, uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world && T > 0 && Vl > 0, "vp_cross_entropy: bad arguments");
  MLF_REQUIRE(ld % 8 == 0 && Vl <= ld && (reinterpret_cast<uintptr_t>(logits) & 15) == 0, "vp_cross_entropy: rows must be 16-byte aligned");
  MLF_REQUIRE(!do_sync || (pads != nullptr && state != nullptr), "vp_cross_entropy: synchronised form needs pads and state");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  long long vc = vocab - lo;
  const int valid_cols = (int)(vc < 0 ? 0 : (vc > Vl ? Vl : vc));
  const int grid = T < sm_count() * 8 ? T : sm_count() * 8;
  vp_ce_stats_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, targets, T, valid_cols, lo,
                                           static_cast<VpStat*>(stats[rank]), device_status_word());
  count_launch();
  // the synchronised form keeps its grid within one wave so that every CTA's wait on the peers ends together
  const int grid2 = do_sync ? (T < sm_count() * 4 ? T : sm_count() * 4) : grid;
  vp_ce_grad_kernel<<<grid2, 256, 0, st>>>(static_cast<__nv_bfloat16*>(logits), ld, Vl, targets, T, valid_cols, lo, vocab,
                                           to_peers(stats, world), pads ? to_peers(pads, world) : PeerPtrs{}, static_cast<SyncState*>(state),
                                           world, rank, do_sync, loss_rows, loss_sum, gscale, gscale_ptr, loss_weight, device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// The two steps of mlf_vp_cross_entropy as separate calls, for callers that exchange the statistics themselves
// (a process-group all-gather between the two).
MLF_API int mlf_vp_ce_stats(const void* logits, long long ld, int Vl, const long long* targets, int T, long long lo, long long vocab,
                            void* stats, uint64_t stream) {
  MLF_REQUIRE(T > 0 && Vl > 0 && ld % 8 == 0 && Vl <= ld && stats != nullptr, "vp_ce_stats: bad arguments");
  long long vc = vocab - lo;
  const int valid_cols = (int)(vc < 0 ? 0 : (vc > Vl ? Vl : vc));
  const int grid = T < sm_count() * 8 ? T : sm_count() * 8;
  vp_ce_stats_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(logits), ld, targets, T,
                                                                              valid_cols, lo, static_cast<VpStat*>(stats),
                                                                              device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
MLF_API int mlf_vp_ce_grad(void* logits, long long ld, int Vl, const long long* targets, int T, long long lo, long long vocab,
                           void* const* stats, void* const* pads, void* state, int world, int rank, int do_sync, float* loss_rows,
                           float* loss_sum, float gscale, const float* gscale_ptr, float loss_weight, uint64_t stream) {
  MLF_REQUIRE(world >= 1 && world <= 8 && T > 0 && Vl > 0 && ld % 8 == 0 && Vl <= ld && do_sync == 0, "vp_ce_grad: bad arguments");
  long long vc = vocab - lo;
  const int valid_cols = (int)(vc < 0 ? 0 : (vc > Vl ? Vl : vc));
  const int grid = T < sm_count() * 8 ? T : sm_count() * 8;
  vp_ce_grad_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), ld, Vl, targets, T, valid_cols, lo, vocab, to_peers(stats, world), PeerPtrs{}, nullptr, world, rank,
      0, loss_rows, loss_sum, gscale, gscale_ptr, loss_weight, device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_sum_partials(const void* partial, int world, long long rows, int cols, void* out, long long ldo,
                             const void* bias, const void* residual, long long ldr, uint64_t stream) {
  MLF_REQUIRE(cols % 8 == 0 && ldo % 8 == 0, "sum_partials: cols and pitch must be multiples of 8");
  long long g = (rows * (cols / 8) + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  sum_partials_kernel<<<(int)g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(partial), world, rows, cols, static_cast<__nv_bfloat16*>(out), ldo,
      static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(residual), ldr);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

MLF_API int mlf_sum_partials_sync(const void* partial, void* const* pads, void* state, int world, int rank, long long rows, int cols,
                                  void* out, long long ldo, const void* bias, const void* residual, long long ldr, uint64_t stream) {
  MLF_REQUIRE(cols % 8 == 0 && ldo % 8 == 0, "sum_partials: cols and pitch must be multiples of 8");
  MLF_REQUIRE(world >= 1 && world <= 8 && state != nullptr, "sum_partials_sync: bad arguments");
  long long g = (rows * (cols / 8) + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  sum_partials_sync_kernel<<<(int)g, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      to_peers(pads, world), static_cast<SyncState*>(state), world, rank, static_cast<const __nv_bfloat16*>(partial), rows, cols,
      static_cast<__nv_bfloat16*>(out), ldo, static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(residual), ldr,
      device_status_word());
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// segs: device array of {src, dst, bytes} (bytes multiple of 16).
MLF_API int mlf_peer_copy(const void* segs, int n_segs, int ctas, uint64_t stream) {
  if (n_segs <= 0) return 0;
  if (ctas <= 0) ctas = sm_count() * 2;
  peer_copy_kernel<<<ctas, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(static_cast<const CopySegHost*>(segs), n_segs);
  count_launch();
  MLF_CHECK_CUDA(cudaGetLastError());
  return 0;
}
