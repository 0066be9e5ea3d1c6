// CUDA-runtime side of the device layer: thin, exception-free wrappers.
// Reference behaviour being covered: device.cpp / queue.cpp / notifier.cpp of
// the reference wrap the vendor runtime the same way
// (torch_mlu/csrc/aten/device/device.cpp:67-121, queue.cpp:111-172,
// notifier.cpp:36-112); here the vendor runtime is the CUDA runtime.
#include <cuda_runtime.h>
#include <cstring>
#include "device_api.h"

extern "C" {

int b200_device_count(void) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int b200_set_device(int device) { return (int)cudaSetDevice(device); }
int b200_get_device(int* device) { return (int)cudaGetDevice(device); }
const char* b200_error_string(int err) { return cudaGetErrorString((cudaError_t)err); }
int b200_get_last_error(void) { return (int)cudaGetLastError(); }

int b200_device_props(int device, B200DeviceProps* out) {
  cudaDeviceProp p;
  cudaError_t e = cudaGetDeviceProperties(&p, device);
  if (e != cudaSuccess) return (int)e;
  std::memset(out, 0, sizeof(*out));
  std::strncpy(out->name, p.name, sizeof(out->name) - 1);
  out->major = p.major;
  out->minor = p.minor;
  out->total_memory = p.totalGlobalMem;
  out->multi_processor_count = p.multiProcessorCount;
  out->max_shared_memory_per_block_optin = (int)p.sharedMemPerBlockOptin;
  out->l2_cache_size = p.l2CacheSize;
  int khz = 0;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device);
  out->clock_rate_khz = khz;
  return 0;
}

int b200_device_synchronize(void) { return (int)cudaDeviceSynchronize(); }

int b200_runtime_version(int* runtime, int* driver) {
  cudaError_t e = cudaRuntimeGetVersion(runtime);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaDriverGetVersion(driver);
}

int b200_malloc(void** ptr, size_t bytes) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) cudaGetLastError();  // clear the sticky OOM so a retry can succeed
  return (int)e;
}
int b200_free(void* ptr) { return (int)cudaFree(ptr); }
int b200_mem_info(size_t* f, size_t* t) { return (int)cudaMemGetInfo(f, t); }
int b200_host_alloc(void** ptr, size_t bytes) { return (int)cudaHostAlloc(ptr, bytes, cudaHostAllocPortable); }
int b200_host_free(void* ptr) { return (int)cudaFreeHost(ptr); }

int b200_memcpy_async(void* dst, const void* src, size_t bytes, int kind, void* stream) {
  cudaMemcpyKind k = cudaMemcpyDefault;
  switch (kind) {
    case B200_MEMCPY_H2D: k = cudaMemcpyHostToDevice; break;
    case B200_MEMCPY_D2H: k = cudaMemcpyDeviceToHost; break;
    case B200_MEMCPY_D2D: k = cudaMemcpyDeviceToDevice; break;
    default: k = cudaMemcpyDefault; break;
  }
  return (int)cudaMemcpyAsync(dst, src, bytes, k, (cudaStream_t)stream);
}

int b200_memcpy_peer_async(void* dst, int dst_dev, const void* src, int src_dev, size_t bytes, void* stream) {
  return (int)cudaMemcpyPeerAsync(dst, dst_dev, src, src_dev, bytes, (cudaStream_t)stream);
}

int b200_memset_async(void* dst, int value, size_t bytes, void* stream) {
  return (int)cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream);
}

int b200_stream_create(void** stream, int priority) {
  cudaStream_t s;
  cudaError_t e = cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, priority);
  *stream = (void*)s;
  return (int)e;
}
int b200_graph_begin_capture(void* stream) {
  return (int)cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeRelaxed);
}
int b200_graph_end_capture(void* stream, void** exec, int* num_nodes) {
  *exec = nullptr;
  if (num_nodes) *num_nodes = 0;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture((cudaStream_t)stream, &graph);
  if (e != cudaSuccess || !graph) {
    cudaGetLastError();  // an invalidated capture leaves a sticky-looking (but recoverable) error behind
    return (int)(e != cudaSuccess ? e : cudaErrorStreamCaptureInvalidated);
  }
  size_t n = 0;
  cudaGraphGetNodes(graph, nullptr, &n);
  if (num_nodes) *num_nodes = (int)n;
  cudaGraphExec_t ex = nullptr;
  e = cudaGraphInstantiate(&ex, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return (int)e;
  *exec = (void*)ex;
  return 0;
}
int b200_graph_launch(void* exec, void* stream) { return (int)cudaGraphLaunch((cudaGraphExec_t)exec, (cudaStream_t)stream); }
int b200_graph_destroy(void* exec) { return (int)cudaGraphExecDestroy((cudaGraphExec_t)exec); }
int b200_stream_is_capturing(void* stream, int* capturing) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  cudaError_t e = cudaStreamIsCapturing((cudaStream_t)stream, &st);
  *capturing = st == cudaStreamCaptureStatusActive ? 1 : 0;
  return (int)e;
}
int b200_stream_destroy(void* stream) { return (int)cudaStreamDestroy((cudaStream_t)stream); }
int b200_stream_synchronize(void* stream) { return (int)cudaStreamSynchronize((cudaStream_t)stream); }
int b200_stream_query(void* stream) {
  cudaError_t e = cudaStreamQuery((cudaStream_t)stream);
  if (e == cudaSuccess) return 0;
  if (e == cudaErrorNotReady) { cudaGetLastError(); return 1; }
  return -(int)e;
}
int b200_stream_wait_event(void* stream, void* event) {
  return (int)cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0);
}

int b200_event_create(void** event, int enable_timing) {
  cudaEvent_t ev;
  cudaError_t e = cudaEventCreateWithFlags(&ev, enable_timing ? cudaEventDefault : cudaEventDisableTiming);
  *event = (void*)ev;
  return (int)e;
}
int b200_event_destroy(void* event) { return (int)cudaEventDestroy((cudaEvent_t)event); }
int b200_event_record(void* event, void* stream) { return (int)cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream); }
int b200_event_synchronize(void* event) { return (int)cudaEventSynchronize((cudaEvent_t)event); }
int b200_event_query(void* event) {
  cudaError_t e = cudaEventQuery((cudaEvent_t)event);
  if (e == cudaSuccess) return 0;
  if (e == cudaErrorNotReady) { cudaGetLastError(); return 1; }
  return -(int)e;
}
int b200_event_elapsed_ms(void* start, void* end, float* ms) {
  return (int)cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)end);
}

int b200_can_access_peer(int device, int peer, int* can) { return (int)cudaDeviceCanAccessPeer(can, device, peer); }
int b200_enable_peer_access(int peer) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
  return (int)e;
}

int b200_ipc_get_handle(void* ptr, char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e == cudaSuccess) std::memcpy(handle, &h, 64);
  return (int)e;
}
int b200_ipc_open_handle(const char handle[64], void** ptr) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
int b200_ipc_close_handle(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }

int b200_host_alloc_mapped(void** host_ptr, void** dev_ptr, size_t bytes) {
  cudaError_t e = cudaHostAlloc(host_ptr, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) return (int)e;
  std::memset(*host_ptr, 0, bytes);
  return (int)cudaHostGetDevicePointer(dev_ptr, *host_ptr, 0);
}

}  // extern "C"

// ---- device-side error flag (one int per device, file-scope) ----------------------
#include "tma_util.cuh"
#include "kernels_api.h"
__device__ int g_b200_error_flag;
namespace b200 {
int* error_flag_ptr() {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_b200_error_flag) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}
}  // namespace b200
extern "C" int b200_read_and_clear_error_flag(int* value) {
  int* p = b200::error_flag_ptr();
  if (!p) return (int)cudaErrorInvalidDevice;
  cudaError_t e = cudaMemcpy(value, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return (int)e;
  if (*value != 0) {
    int zero = 0;
    e = cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return (int)e;
}
