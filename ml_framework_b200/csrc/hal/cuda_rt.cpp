// Native binding of the CUDA runtime calls the framework's HAL exposes: devices, memory, streams,
// events and graphs (capture, instantiate, launch, node inspection). The reference binds the same
// 23 entry points through P/Invoke (src/MLFramework/HAL/CUDA/CudaApi.cs:19-184, up to
// CudaGraphGetNodes :184) against a library that is not in its tree; here they are a C ABI over
// libcudart, reached from Python with ctypes (ml_framework_b200/hal/cuda_rt.py). Every function
// returns 0 on success or a negative code with a message in mlf_last_error(); handles cross the
// ABI as 64-bit integers.
//
// Graph inspection is what the validator works on: after a capture the node list of the real
// cudaGraph_t is read back with its node types (kernel, memcpy, memset, host callback, memory
// allocation / free, event wait / record, child graph), so validation rules apply to what the capture
// recorded rather than what a caller declares.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <vector>

#include "../common/host.h"

using namespace mlf;

// ---- devices ---------------------------------------------------------------------------------
MLF_API int mlf_rt_device_count(int* n) {
  MLF_REQUIRE(n != nullptr, "rt_device_count: null result");
  cudaError_t e = cudaGetDeviceCount(n);
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) {
    *n = 0;
    (void)cudaGetLastError();
    return 0;
  }
  MLF_CHECK_CUDA(e);
  return 0;
}
MLF_API int mlf_rt_set_device(int dev) {
  MLF_CHECK_CUDA(cudaSetDevice(dev));
  return 0;
}
MLF_API int mlf_rt_get_device(int* dev) {
  MLF_CHECK_CUDA(cudaGetDevice(dev));
  return 0;
}
// props: [0] multiprocessors, [1] compute major, [2] compute minor, [3] total memory MiB,
// [4] max shared memory per block (opt-in) bytes, [5] L2 bytes, [6] SM clock kHz, [7] memory bus bits.
MLF_API int mlf_rt_device_properties(int dev, long long* props8, char* name, int name_len) {
  cudaDeviceProp p;
  MLF_CHECK_CUDA(cudaGetDeviceProperties(&p, dev));
  int clk = 0;
  cudaDeviceGetAttribute(&clk, cudaDevAttrClockRate, dev);
  props8[0] = p.multiProcessorCount;
  props8[1] = p.major;
  props8[2] = p.minor;
  props8[3] = (long long)(p.totalGlobalMem >> 20);
  props8[4] = (long long)p.sharedMemPerBlockOptin;
  props8[5] = p.l2CacheSize;
  props8[6] = clk;
  props8[7] = p.memoryBusWidth;
  if (name && name_len > 0) {
    strncpy(name, p.name, (size_t)name_len - 1);
    name[name_len - 1] = 0;
  }
  return 0;
}
MLF_API int mlf_rt_device_synchronize() {
  MLF_CHECK_CUDA(cudaDeviceSynchronize());
  return 0;
}
MLF_API int mlf_rt_mem_info(long long* free_bytes, long long* total_bytes) {
  size_t f = 0, t = 0;
  MLF_CHECK_CUDA(cudaMemGetInfo(&f, &t));
  *free_bytes = (long long)f;
  *total_bytes = (long long)t;
  return 0;
}

// ---- memory ----------------------------------------------------------------------------------
MLF_API int mlf_rt_malloc(long long bytes, uint64_t* ptr) {
  MLF_REQUIRE(bytes > 0 && ptr, "rt_malloc: bad arguments");
  void* p = nullptr;
  MLF_CHECK_CUDA(cudaMalloc(&p, (size_t)bytes));
  *ptr = reinterpret_cast<uint64_t>(p);
  return 0;
}
MLF_API int mlf_rt_free(uint64_t ptr) {
  MLF_CHECK_CUDA(cudaFree(reinterpret_cast<void*>(ptr)));
  return 0;
}
MLF_API int mlf_rt_malloc_host(long long bytes, uint64_t* ptr) {
  MLF_REQUIRE(bytes > 0 && ptr, "rt_malloc_host: bad arguments");
  void* p = nullptr;
  MLF_CHECK_CUDA(cudaMallocHost(&p, (size_t)bytes));
  *ptr = reinterpret_cast<uint64_t>(p);
  return 0;
}
MLF_API int mlf_rt_free_host(uint64_t ptr) {
  MLF_CHECK_CUDA(cudaFreeHost(reinterpret_cast<void*>(ptr)));
  return 0;
}
// kind: 0 host->host, 1 host->device, 2 device->host, 3 device->device, 4 default (by address)
MLF_API int mlf_rt_memcpy(uint64_t dst, uint64_t src, long long bytes, int kind, uint64_t stream, int async) {
  MLF_REQUIRE(kind >= 0 && kind <= 4 && bytes >= 0, "rt_memcpy: bad arguments");
  if (bytes == 0) return 0;
  cudaMemcpyKind k = static_cast<cudaMemcpyKind>(kind);
  if (async)
    MLF_CHECK_CUDA(cudaMemcpyAsync(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), (size_t)bytes, k,
                                   reinterpret_cast<cudaStream_t>(stream)));
  else
    MLF_CHECK_CUDA(cudaMemcpy(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), (size_t)bytes, k));
  return 0;
}
MLF_API int mlf_rt_memset(uint64_t dst, int value, long long bytes, uint64_t stream, int async) {
  if (bytes <= 0) return 0;
  if (async)
    MLF_CHECK_CUDA(cudaMemsetAsync(reinterpret_cast<void*>(dst), value, (size_t)bytes, reinterpret_cast<cudaStream_t>(stream)));
  else
    MLF_CHECK_CUDA(cudaMemset(reinterpret_cast<void*>(dst), value, (size_t)bytes));
  return 0;
}

// ---- streams and events ------------------------------------------------------------------------
MLF_API int mlf_rt_stream_create(int non_blocking, int priority, uint64_t* stream) {
  cudaStream_t s = nullptr;
  MLF_CHECK_CUDA(cudaStreamCreateWithPriority(&s, non_blocking ? cudaStreamNonBlocking : cudaStreamDefault, priority));
  *stream = reinterpret_cast<uint64_t>(s);
  return 0;
}
MLF_API int mlf_rt_stream_destroy(uint64_t stream) {
  MLF_CHECK_CUDA(cudaStreamDestroy(reinterpret_cast<cudaStream_t>(stream)));
  return 0;
}
MLF_API int mlf_rt_stream_synchronize(uint64_t stream) {
  MLF_CHECK_CUDA(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  return 0;
}
// done: 1 when all work queued on the stream has completed
MLF_API int mlf_rt_stream_query(uint64_t stream, int* done) {
  cudaError_t e = cudaStreamQuery(reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaErrorNotReady) {
    *done = 0;
    (void)cudaGetLastError();
    return 0;
  }
  MLF_CHECK_CUDA(e);
  *done = 1;
  return 0;
}
MLF_API int mlf_rt_stream_wait_event(uint64_t stream, uint64_t event) {
  MLF_CHECK_CUDA(cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(stream), reinterpret_cast<cudaEvent_t>(event), 0));
  return 0;
}
MLF_API int mlf_rt_event_create(int timing, uint64_t* event) {
  cudaEvent_t e = nullptr;
  MLF_CHECK_CUDA(cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming));
  *event = reinterpret_cast<uint64_t>(e);
  return 0;
}
MLF_API int mlf_rt_event_destroy(uint64_t event) {
  MLF_CHECK_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
  return 0;
}
MLF_API int mlf_rt_event_record(uint64_t event, uint64_t stream) {
  MLF_CHECK_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), reinterpret_cast<cudaStream_t>(stream)));
  return 0;
}
MLF_API int mlf_rt_event_synchronize(uint64_t event) {
  MLF_CHECK_CUDA(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(event)));
  return 0;
}
MLF_API int mlf_rt_event_query(uint64_t event, int* done) {
  cudaError_t e = cudaEventQuery(reinterpret_cast<cudaEvent_t>(event));
  if (e == cudaErrorNotReady) {
    *done = 0;
    (void)cudaGetLastError();
    return 0;
  }
  MLF_CHECK_CUDA(e);
  *done = 1;
  return 0;
}
MLF_API int mlf_rt_event_elapsed_ms(uint64_t start, uint64_t end, float* ms) {
  MLF_CHECK_CUDA(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start), reinterpret_cast<cudaEvent_t>(end)));
  return 0;
}

// ---- graphs ----------------------------------------------------------------------------------
// mode: 0 global, 1 thread-local, 2 relaxed
MLF_API int mlf_rt_stream_begin_capture(uint64_t stream, int mode) {
  MLF_REQUIRE(mode >= 0 && mode <= 2, "rt_stream_begin_capture: mode must be 0, 1 or 2");
  MLF_CHECK_CUDA(cudaStreamBeginCapture(reinterpret_cast<cudaStream_t>(stream), static_cast<cudaStreamCaptureMode>(mode)));
  return 0;
}
MLF_API int mlf_rt_stream_end_capture(uint64_t stream, uint64_t* graph) {
  cudaGraph_t g = nullptr;
  MLF_CHECK_CUDA(cudaStreamEndCapture(reinterpret_cast<cudaStream_t>(stream), &g));
  MLF_REQUIRE(g != nullptr, "rt_stream_end_capture: the capture was invalidated");
  *graph = reinterpret_cast<uint64_t>(g);
  return 0;
}
MLF_API int mlf_rt_stream_is_capturing(uint64_t stream, int* capturing) {
  cudaStreamCaptureStatus st;
  MLF_CHECK_CUDA(cudaStreamIsCapturing(reinterpret_cast<cudaStream_t>(stream), &st));
  *capturing = st == cudaStreamCaptureStatusActive ? 1 : 0;
  return 0;
}
MLF_API int mlf_rt_graph_instantiate(uint64_t graph, uint64_t* exec) {
  cudaGraphExec_t x = nullptr;
  MLF_CHECK_CUDA(cudaGraphInstantiate(&x, reinterpret_cast<cudaGraph_t>(graph), 0));
  *exec = reinterpret_cast<uint64_t>(x);
  return 0;
}
MLF_API int mlf_rt_graph_launch(uint64_t exec, uint64_t stream) {
  MLF_CHECK_CUDA(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(exec), reinterpret_cast<cudaStream_t>(stream)));
  return 0;
}
MLF_API int mlf_rt_graph_destroy(uint64_t graph) {
  MLF_CHECK_CUDA(cudaGraphDestroy(reinterpret_cast<cudaGraph_t>(graph)));
  return 0;
}
MLF_API int mlf_rt_graph_exec_destroy(uint64_t exec) {
  MLF_CHECK_CUDA(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(exec)));
  return 0;
}
// Node census of a graph. types[i] receives the cudaGraphNodeType of node i for i < capacity;
// *count receives the number of nodes. Child graphs are not expanded: they count as one node of
// type cudaGraphNodeTypeGraph.
MLF_API int mlf_rt_graph_get_nodes(uint64_t graph, int* types, int capacity, int* count) {
  MLF_REQUIRE(count != nullptr, "rt_graph_get_nodes: null count");
  cudaGraph_t g = reinterpret_cast<cudaGraph_t>(graph);
  size_t n = 0;
  MLF_CHECK_CUDA(cudaGraphGetNodes(g, nullptr, &n));
  *count = (int)n;
  if (!types || capacity <= 0 || n == 0) return 0;
  std::vector<cudaGraphNode_t> nodes(n);
  MLF_CHECK_CUDA(cudaGraphGetNodes(g, nodes.data(), &n));
  for (size_t i = 0; i < n && (int)i < capacity; ++i) {
    cudaGraphNodeType t;
    MLF_CHECK_CUDA(cudaGraphNodeGetType(nodes[i], &t));
    types[i] = (int)t;
  }
  return 0;
}
