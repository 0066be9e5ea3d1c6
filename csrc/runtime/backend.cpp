#include "backend.h"

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "../device/device_api.h"
#include "log.h"

namespace catch_b200 {

namespace {

// ---------------------------------------------------------------- CUDA backend
class CudaBackend final : public Backend {
 public:
  bool is_hostsim() const override { return false; }
  const char* name() const override { return "cuda"; }

  int device_count() override {
    static int n = b200_device_count();
    return n;
  }
  void set_device(int d) override { B200_DEVICE_CHECK(b200_set_device(d)); }
  int get_device() override {
    int d = 0;
    B200_DEVICE_CHECK(b200_get_device(&d));
    return d;
  }
  void device_synchronize() override { B200_DEVICE_CHECK(b200_device_synchronize()); }
  DeviceProp device_props(int device) override {
    B200DeviceProps p;
    B200_DEVICE_CHECK(b200_device_props(device, &p));
    DeviceProp out;
    out.name = p.name;
    out.major = p.major;
    out.minor = p.minor;
    out.total_memory = p.total_memory;
    out.multi_processor_count = p.multi_processor_count;
    out.max_shared_memory_per_block_optin = p.max_shared_memory_per_block_optin;
    out.l2_cache_size = p.l2_cache_size;
    return out;
  }
  void versions(int* rt, int* drv) override { B200_DEVICE_CHECK(b200_runtime_version(rt, drv)); }

  int try_malloc(void** p, size_t n) override { return b200_malloc(p, n); }
  void free(void* p) override { B200_DEVICE_WARN(b200_free(p)); }
  void mem_info(size_t* f, size_t* t) override { B200_DEVICE_CHECK(b200_mem_info(f, t)); }
  int try_host_alloc(void** p, size_t n) override { return b200_host_alloc(p, n); }
  void host_free(void* p) override { B200_DEVICE_WARN(b200_host_free(p)); }

  void memcpy_async(void* dst, const void* src, size_t n, CopyKind k, void* s) override {
    if (n == 0) return;
    B200_DEVICE_CHECK(b200_memcpy_async(dst, src, n, static_cast<int>(k), s));
  }
  void memcpy_peer_async(void* dst, int dd, const void* src, int sd, size_t n, void* s) override {
    if (n == 0) return;
    B200_DEVICE_CHECK(b200_memcpy_peer_async(dst, dd, src, sd, n, s));
  }
  void memset_async(void* dst, int v, size_t n, void* s) override {
    if (n == 0) return;
    B200_DEVICE_CHECK(b200_memset_async(dst, v, n, s));
  }

  void* stream_create(int prio) override {
    void* s = nullptr;
    B200_DEVICE_CHECK(b200_stream_create(&s, prio));
    return s;
  }
  void stream_destroy(void* s) override { B200_DEVICE_WARN(b200_stream_destroy(s)); }
  void stream_synchronize(void* s) override { B200_DEVICE_CHECK(b200_stream_synchronize(s)); }
  bool stream_query(void* s) override {
    int r = b200_stream_query(s);
    TORCH_CHECK(r >= 0, "b200 stream query failed: ", b200_error_string(-r));
    return r == 0;
  }
  void stream_wait_event(void* s, void* e) override { B200_DEVICE_CHECK(b200_stream_wait_event(s, e)); }

  bool supports_graphs() const override { return true; }
  void graph_begin_capture(void* s) override { B200_DEVICE_CHECK(b200_graph_begin_capture(s)); }
  void* graph_end_capture(void* s, int* num_nodes) override {
    void* exec = nullptr;
    const int rc = b200_graph_end_capture(s, &exec, num_nodes);
    if (rc != 0) {
      B200LOG(DBG) << "graph capture did not produce a graph: " << b200_error_string(rc);
      return nullptr;
    }
    return exec;
  }
  void graph_launch(void* exec, void* s) override { B200_DEVICE_CHECK(b200_graph_launch(exec, s)); }
  void graph_destroy(void* exec) override { B200_DEVICE_WARN(b200_graph_destroy(exec)); }
  void* event_create(bool timing) override {
    void* e = nullptr;
    B200_DEVICE_CHECK(b200_event_create(&e, timing ? 1 : 0));
    return e;
  }
  void event_destroy(void* e) override { B200_DEVICE_WARN(b200_event_destroy(e)); }
  void event_record(void* e, void* s) override { B200_DEVICE_CHECK(b200_event_record(e, s)); }
  void event_synchronize(void* e) override { B200_DEVICE_CHECK(b200_event_synchronize(e)); }
  bool event_query(void* e) override {
    int r = b200_event_query(e);
    TORCH_CHECK(r >= 0, "b200 event query failed: ", b200_error_string(-r));
    return r == 0;
  }
  float event_elapsed_ms(void* a, void* b) override {
    float ms = 0.f;
    B200_DEVICE_CHECK(b200_event_elapsed_ms(a, b, &ms));
    return ms;
  }
};

// ------------------------------------------------------------ host simulation
// Work submitted to a simulated queue completes before the call returns, so a
// queue is always idle and an event is "done" as soon as it has been recorded.
struct SimStream {
  int device;
};
struct SimEvent {
  bool recorded = false;
  std::chrono::steady_clock::time_point t;
};

class HostSimBackend final : public Backend {
 public:
  explicit HostSimBackend(int ndev) : ndev_(ndev) {}
  bool is_hostsim() const override { return true; }
  const char* name() const override { return "hostsim"; }

  int device_count() override { return ndev_; }
  void set_device(int d) override {
    TORCH_CHECK(d >= 0 && d < ndev_, "b200(hostsim): invalid device ordinal ", d);
    current() = d;
  }
  int get_device() override { return current(); }
  void device_synchronize() override {}
  DeviceProp device_props(int device) override {
    TORCH_CHECK(device >= 0 && device < ndev_, "b200(hostsim): invalid device ordinal ", device);
    DeviceProp p;
    p.name = "B200 (host simulation)";
    p.major = 10;
    p.minor = 0;
    p.total_memory = kSimMemory;
    p.multi_processor_count = 148;
    p.max_shared_memory_per_block_optin = 227 * 1024;
    p.l2_cache_size = 126 * 1024 * 1024;
    return p;
  }
  void versions(int* rt, int* drv) override {
    *rt = 0;
    *drv = 0;
  }

  int try_malloc(void** p, size_t n) override {
    if (used_.load() + n > limit_.load()) {
      *p = nullptr;
      return 2;  // same numeric value as cudaErrorMemoryAllocation
    }
    void* q = nullptr;
    if (posix_memalign(&q, 512, n ? n : 512) != 0) {
      *p = nullptr;
      return 2;
    }
    used_ += n;
    {
      std::lock_guard<std::mutex> g(mu_);
      sizes_.emplace_back(q, n);
    }
    *p = q;
    return 0;
  }
  void free(void* p) override {
    {
      std::lock_guard<std::mutex> g(mu_);
      for (size_t i = 0; i < sizes_.size(); ++i) {
        if (sizes_[i].first == p) {
          used_ -= sizes_[i].second;
          sizes_[i] = sizes_.back();
          sizes_.pop_back();
          break;
        }
      }
    }
    std::free(p);
  }
  void mem_info(size_t* f, size_t* t) override {
    *t = limit_.load();
    size_t u = used_.load();
    *f = u > *t ? 0 : *t - u;
  }
  int try_host_alloc(void** p, size_t n) override {
    return posix_memalign(p, 4096, n ? n : 4096) == 0 ? 0 : 2;
  }
  void host_free(void* p) override { std::free(p); }

  void memcpy_async(void* dst, const void* src, size_t n, CopyKind, void*) override {
    if (n) std::memmove(dst, src, n);
  }
  void memcpy_peer_async(void* dst, int, const void* src, int, size_t n, void*) override {
    if (n) std::memmove(dst, src, n);
  }
  void memset_async(void* dst, int v, size_t n, void*) override {
    if (n) std::memset(dst, v, n);
  }

  void* stream_create(int) override { return new SimStream{current()}; }
  void stream_destroy(void* s) override { delete static_cast<SimStream*>(s); }
  void stream_synchronize(void*) override {}
  bool stream_query(void*) override { return true; }
  void stream_wait_event(void*, void*) override {}

  // Simulated work runs when it is submitted, so there is nothing to capture or replay.
  bool supports_graphs() const override { return false; }
  void graph_begin_capture(void*) override { TORCH_CHECK(false, "b200(hostsim): graph capture needs a device"); }
  void* graph_end_capture(void*, int*) override { return nullptr; }
  void graph_launch(void*, void*) override { TORCH_CHECK(false, "b200(hostsim): graph replay needs a device"); }
  void graph_destroy(void*) override {}
  void* event_create(bool) override { return new SimEvent(); }
  void event_destroy(void* e) override { delete static_cast<SimEvent*>(e); }
  void event_record(void* e, void*) override {
    auto* ev = static_cast<SimEvent*>(e);
    ev->recorded = true;
    ev->t = std::chrono::steady_clock::now();
  }
  void event_synchronize(void*) override {}
  bool event_query(void*) override { return true; }
  float event_elapsed_ms(void* a, void* b) override {
    auto* ea = static_cast<SimEvent*>(a);
    auto* eb = static_cast<SimEvent*>(b);
    TORCH_CHECK(ea->recorded && eb->recorded, "b200: both notifiers must be placed before elapsed_time");
    return std::chrono::duration<float, std::milli>(eb->t - ea->t).count();
  }

  // Test hook: shrink the simulated memory so OOM paths can be exercised.
  void set_limit(size_t bytes) { limit_ = bytes; }

 private:
  static constexpr size_t kSimMemory = size_t(8) << 30;
  static int& current() {
    thread_local int d = 0;
    return d;
  }
  int ndev_;
  std::atomic<size_t> used_{0};
  std::atomic<size_t> limit_{kSimMemory};
  std::mutex mu_;
  std::vector<std::pair<void*, size_t>> sizes_;
};

HostSimBackend* g_hostsim = nullptr;

}  // namespace

Backend& backend() {
  static std::unique_ptr<Backend> inst = [] {
    const std::string& want = flags().backend;
    std::unique_ptr<Backend> b;
    if (want == "hostsim") {
      g_hostsim = new HostSimBackend(flags().hostsim_devices);
      b.reset(g_hostsim);
    } else if (want == "cuda") {
      b = std::make_unique<CudaBackend>();
    } else {
      if (b200_device_count() > 0) {
        b = std::make_unique<CudaBackend>();
      } else {
        g_hostsim = new HostSimBackend(flags().hostsim_devices);
        b.reset(g_hostsim);
      }
    }
    B200LOG(INFO) << "b200 backend: " << b->name() << ", devices: " << b->device_count();
    return b;
  }();
  return *inst;
}

// Exposed for tests (declared in device.h).
void hostsim_set_memory_limit(size_t bytes) {
  backend();
  TORCH_CHECK(g_hostsim != nullptr, "hostsim_set_memory_limit needs the host-simulated backend");
  g_hostsim->set_limit(bytes);
}

}  // namespace catch_b200
