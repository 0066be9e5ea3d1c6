// Profiler integration for the b200 device.
//
// The reference patches PyTorch to add a ProfilerState::MLU and collects device
// kernel times with a vendor tracer (torch_mlu/csrc/aten/profile/profile_mlu.cpp:
// 76-329).  Here the stock profiler's PrivateUse1 stub interface is implemented
// with notifiers: torch.autograd.profiler.profile(use_device="blackwell") records a
// notifier at the start and end of every op on the current queue, and the device
// columns of .table() / key_averages() / export_chrome_trace() come from
// elapsed_time between them.  Memory events are reported by the caching allocator
// through c10::reportMemoryUsageToProfiler.
#include <torch/csrc/profiler/stubs/base.h>
#include <c10/util/ApproximateClock.h>

#include "device.h"
#include "notifier.h"

namespace catch_b200 {
namespace {

struct B200ProfilerStubs final : public torch::profiler::impl::ProfilerStubs {
  void record(c10::DeviceIndex* device, torch::profiler::impl::ProfilerVoidEventStub* event, int64_t* cpu_ns) const override {
    const int dev = current_device();
    if (device) *device = static_cast<c10::DeviceIndex>(dev);
    auto n = std::make_shared<Notifier>(/*enable_timing=*/true);
    Queue q = getCurrentQueue(dev);
    if (cpu_ns) *cpu_ns = c10::getTime();
    n->place(q);
    *event = std::static_pointer_cast<void>(n);
  }
  float elapsed(const torch::profiler::impl::ProfilerVoidEventStub* a,
                const torch::profiler::impl::ProfilerVoidEventStub* b) const override {
    auto na = std::static_pointer_cast<Notifier>(*a);
    auto nb = std::static_pointer_cast<Notifier>(*b);
    na->synchronize();
    nb->synchronize();
    return na->elapsed_time(*nb) * 1000.0f;  // microseconds
  }
  void mark(const char*) const override {}
  void rangePush(const char*) const override {}
  void rangePop() const override {}
  bool enabled() const override { return true; }
  void onEachDevice(std::function<void(int)> op) const override {
    const int prev = current_device();
    for (int d = 0; d < device_count(); ++d) {
      DeviceSwitch sw(d);
      op(d);
    }
    (void)prev;
  }
  void synchronize() const override { catch_b200::synchronize(-1); }
};

struct RegisterStubs {
  RegisterStubs() {
    static B200ProfilerStubs stubs;
    torch::profiler::impl::registerPrivateUse1Methods(&stubs);
  }
};
RegisterStubs g_register;

}  // namespace
}  // namespace catch_b200
