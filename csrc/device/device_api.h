// C ABI of the device layer (libcatch_b200_device.so).
//
// Everything that touches the CUDA runtime or launches a kernel lives behind
// this header and is compiled by nvcc for sm_100a only.  The host runtime
// (allocator, queues, notifiers, operators, process group) is plain C++ and
// talks to the GPU exclusively through these functions, so it can be swapped
// for the host-simulated backend when no GPU is present.
//
// Conventions: every function returns 0 on success or a CUDA error code
// (see b200_error_string).  Streams and events are opaque pointers.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

typedef struct B200DeviceProps {
  char name[256];
  int major;
  int minor;
  size_t total_memory;
  int multi_processor_count;
  int max_shared_memory_per_block_optin;
  int l2_cache_size;
  int clock_rate_khz;
} B200DeviceProps;

enum { B200_MEMCPY_H2D = 1, B200_MEMCPY_D2H = 2, B200_MEMCPY_D2D = 3, B200_MEMCPY_H2H = 0 };

// ---- runtime ---------------------------------------------------------------
B200_API int b200_device_count(void);
B200_API int b200_set_device(int device);
B200_API int b200_get_device(int* device);
B200_API const char* b200_error_string(int err);
B200_API int b200_get_last_error(void);
B200_API int b200_device_props(int device, B200DeviceProps* out);
B200_API int b200_device_synchronize(void);
B200_API int b200_runtime_version(int* runtime, int* driver);

B200_API int b200_malloc(void** ptr, size_t bytes);
B200_API int b200_free(void* ptr);
B200_API int b200_mem_info(size_t* free_bytes, size_t* total_bytes);
B200_API int b200_host_alloc(void** ptr, size_t bytes);
B200_API int b200_host_free(void* ptr);
B200_API int b200_memcpy_async(void* dst, const void* src, size_t bytes, int kind, void* stream);
B200_API int b200_memcpy_peer_async(void* dst, int dst_dev, const void* src, int src_dev, size_t bytes, void* stream);
B200_API int b200_memset_async(void* dst, int value, size_t bytes, void* stream);

B200_API int b200_stream_create(void** stream, int priority);
B200_API int b200_stream_destroy(void* stream);
B200_API int b200_stream_synchronize(void* stream);
B200_API int b200_stream_query(void* stream);  // 0 = done, 1 = busy, <0 = -error
B200_API int b200_stream_wait_event(void* stream, void* event);

// Stream capture into an executable graph.  Capture runs in relaxed mode (the caching allocator may still ask the
// driver for memory while a queue is capturing).  b200_graph_end_capture instantiates the captured graph; when
// the capture was invalidated (a synchronising call inside it) it returns the error and leaves *exec null.
B200_API int b200_graph_begin_capture(void* stream);
B200_API int b200_graph_end_capture(void* stream, void** exec, int* num_nodes);
B200_API int b200_graph_launch(void* exec, void* stream);
B200_API int b200_graph_destroy(void* exec);
B200_API int b200_stream_is_capturing(void* stream, int* capturing);

B200_API int b200_event_create(void** event, int enable_timing);
B200_API int b200_event_destroy(void* event);
B200_API int b200_event_record(void* event, void* stream);
B200_API int b200_event_synchronize(void* event);
B200_API int b200_event_query(void* event);  // 0 = done, 1 = busy, <0 = -error
B200_API int b200_event_elapsed_ms(void* start, void* end, float* ms);

B200_API int b200_can_access_peer(int device, int peer, int* can);
B200_API int b200_enable_peer_access(int peer);
// 64-byte IPC handles for exchanging symmetric buffers between ranks.
B200_API int b200_ipc_get_handle(void* ptr, char handle[64]);
B200_API int b200_ipc_open_handle(const char handle[64], void** ptr);
B200_API int b200_ipc_close_handle(void* ptr);
// Symmetric memory through the virtual-memory-management API (vmm.cu): allocations that are shared as POSIX
// file descriptors and bound to an NVSwitch multicast object, so that one address names the same offset of
// every rank's buffer (multimem.ld_reduce / multimem.st).  b200_vmm_import / b200_mc_import close the descriptor.
B200_API int b200_vmm_multicast_supported(int device, int* supported);
B200_API int b200_vmm_round_size(int device, int ndevices, size_t bytes, size_t* rounded);
B200_API int b200_vmm_alloc(size_t bytes, int device, void** ptr, unsigned long long* handle, int* fd);
B200_API int b200_vmm_import(int fd, size_t bytes, int device, void** ptr, unsigned long long* handle);
B200_API int b200_vmm_release(void* ptr, size_t bytes, unsigned long long handle);
B200_API int b200_mc_create(int ndevices, size_t bytes, unsigned long long* mc, int* fd);
B200_API int b200_mc_import(int fd, unsigned long long* mc);
B200_API int b200_mc_add_device(unsigned long long mc, int device);
B200_API int b200_mc_bind(unsigned long long mc, unsigned long long mem_handle, size_t bytes);
B200_API int b200_mc_map(unsigned long long mc, size_t bytes, int device, void** ptr);
B200_API int b200_mc_release(void* ptr, size_t bytes, unsigned long long mc, int device, int bound);
// Host-mapped (zero-copy) status words: kernels write, the host polls.
B200_API int b200_host_alloc_mapped(void** host_ptr, void** dev_ptr, size_t bytes);

#ifdef __cplusplus
}
#endif
