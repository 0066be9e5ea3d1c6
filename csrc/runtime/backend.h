// Backend interface of the host runtime.
//
// Two implementations share every line of the plumbing above them (allocator,
// queues, notifiers, tensor construction, operator registration):
//   * CudaBackend    -- forwards to the device layer (CUDA runtime, sm_100a kernels)
//   * HostSimBackend -- "device memory" is host memory, queues execute inline and
//                       notifiers are host timestamps, so the whole stack runs
//                       on a machine with no GPU.
// The reference has no such mode (all of its tests need hardware); only
// DEFAULT_MLU_DEVICE_NAME skips probing (torch_mlu/csrc/aten/util/common.cpp:55-64).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace catch_b200 {

struct DeviceProp {
  std::string name;
  int major = 0;
  int minor = 0;
  size_t total_memory = 0;
  int multi_processor_count = 0;
  int max_shared_memory_per_block_optin = 0;
  int l2_cache_size = 0;
};

enum class CopyKind : int { H2H = 0, H2D = 1, D2H = 2, D2D = 3 };

class Backend {
 public:
  virtual ~Backend() = default;
  virtual bool is_hostsim() const = 0;
  virtual const char* name() const = 0;

  virtual int device_count() = 0;
  virtual void set_device(int device) = 0;
  virtual int get_device() = 0;
  virtual void device_synchronize() = 0;
  virtual DeviceProp device_props(int device) = 0;
  virtual void versions(int* runtime, int* driver) = 0;

  // Returns an error code instead of throwing so the allocator can retry.
  virtual int try_malloc(void** ptr, size_t bytes) = 0;
  virtual void free(void* ptr) = 0;
  virtual void mem_info(size_t* free_bytes, size_t* total_bytes) = 0;
  virtual int try_host_alloc(void** ptr, size_t bytes) = 0;
  virtual void host_free(void* ptr) = 0;

  virtual void memcpy_async(void* dst, const void* src, size_t bytes, CopyKind kind, void* stream) = 0;
  virtual void memcpy_peer_async(void* dst, int dst_dev, const void* src, int src_dev, size_t bytes, void* stream) = 0;
  virtual void memset_async(void* dst, int value, size_t bytes, void* stream) = 0;

  virtual void* stream_create(int priority) = 0;
  virtual void stream_destroy(void* s) = 0;
  virtual void stream_synchronize(void* s) = 0;
  virtual bool stream_query(void* s) = 0;
  virtual void stream_wait_event(void* s, void* e) = 0;

  // Stream capture (executable graphs).  graph_end_capture returns null when the capture was invalidated.
  virtual bool supports_graphs() const = 0;
  virtual void graph_begin_capture(void* s) = 0;
  virtual void* graph_end_capture(void* s, int* num_nodes) = 0;
  virtual void graph_launch(void* exec, void* s) = 0;
  virtual void graph_destroy(void* exec) = 0;

  virtual void* event_create(bool timing) = 0;
  virtual void event_destroy(void* e) = 0;
  virtual void event_record(void* e, void* s) = 0;
  virtual void event_synchronize(void* e) = 0;
  virtual bool event_query(void* e) = 0;
  virtual float event_elapsed_ms(void* start, void* end) = 0;
};

// Process-wide backend chosen on first use from CATCH_B200_BACKEND
// (auto = CUDA when a device is visible, else host simulation).
Backend& backend();
inline bool hostsim() { return backend().is_hostsim(); }

}  // namespace catch_b200
