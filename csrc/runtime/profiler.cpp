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

#include <atomic>
#include <memory>
#include <mutex>

#include "device.h"
#include "notifier.h"
#include "profiler.h"

#include "graph.h"

namespace catch_b200 {

// ------------------------------------------------------------------------------ kernel trace
namespace {
struct PendingEvent {
  KernelEvent ev;
  std::shared_ptr<Notifier> start, end;
};
std::atomic<bool> g_trace_on{false};
std::mutex g_trace_mu;
std::vector<std::unique_ptr<PendingEvent>> g_trace;
std::vector<std::shared_ptr<Notifier>> g_trace_base(64);   // per device: time zero of the trace
thread_local const char* t_current_op = "";
thread_local std::vector<PendingEvent*> t_range_stack;

std::shared_ptr<Notifier> place_now(int dev) {
  auto n = std::make_shared<Notifier>(/*enable_timing=*/true);
  n->place(getCurrentQueue(dev));
  return n;
}
PendingEvent* new_event(const char* name, int kind) {
  auto pe = std::make_unique<PendingEvent>();
  pe->ev.name = name ? name : "";
  pe->ev.kind = kind;
  pe->ev.device = current_device();
  pe->ev.queue = getCurrentQueue(pe->ev.device).pack();
  pe->ev.cpu_ns = c10::getTime();
  PendingEvent* raw = pe.get();
  std::lock_guard<std::mutex> lk(g_trace_mu);
  if (!g_trace_base[pe->ev.device & 63]) {
    // first event on this device: its time zero sits on the same queue, just before the event
    g_trace_base[pe->ev.device & 63] = place_now(pe->ev.device);
  }
  g_trace.push_back(std::move(pe));
  return raw;
}
// "b200_conv_fprop(&p, scope.stream())" -> "b200_conv_fprop"
std::string launcher_name(const char* expr) {
  std::string s(expr ? expr : "");
  const size_t paren = s.find('(');
  if (paren != std::string::npos) s.resize(paren);
  while (!s.empty() && (s.back() == ' ')) s.pop_back();
  return s;
}
}  // namespace

bool kernel_trace_enabled() { return g_trace_on.load(std::memory_order_relaxed); }
void kernel_trace_start() {
  std::lock_guard<std::mutex> lk(g_trace_mu);
  g_trace.clear();
  for (auto& b : g_trace_base) b.reset();
  g_trace_on.store(true);
}
std::vector<KernelEvent> kernel_trace_stop() {
  g_trace_on.store(false);
  std::vector<std::unique_ptr<PendingEvent>> taken;
  std::vector<std::shared_ptr<Notifier>> base;
  {
    std::lock_guard<std::mutex> lk(g_trace_mu);
    taken.swap(g_trace);
    base = g_trace_base;
    for (auto& b : g_trace_base) b.reset();
  }
  std::vector<KernelEvent> out;
  out.reserve(taken.size());
  for (auto& pe : taken) {
    if (pe->start && (pe->end || pe->ev.kind == 2)) {
      auto& b = base[pe->ev.device & 63];
      pe->start->synchronize();
      if (b) pe->ev.start_us = b->elapsed_time(*pe->start) * 1000.0;
      if (pe->end) {
        pe->end->synchronize();
        pe->ev.dur_us = pe->start->elapsed_time(*pe->end) * 1000.0;
      }
    }
    out.push_back(std::move(pe->ev));
  }
  return out;
}
const char* trace_current_op() { return t_current_op; }
const char* trace_set_current_op(const char* name) {
  const char* prev = t_current_op;
  t_current_op = name ? name : "";
  return prev;
}
void trace_mark(const char* name) {
  if (!kernel_trace_enabled()) return;
  PendingEvent* pe = new_event(name, 2);
  pe->start = place_now(pe->ev.device);
}
void trace_range_push(const char* name) {
  if (!kernel_trace_enabled()) return;
  PendingEvent* pe = new_event(name, 1);
  pe->start = place_now(pe->ev.device);
  t_range_stack.push_back(pe);
}
void trace_range_pop() {
  if (t_range_stack.empty()) return;
  PendingEvent* pe = t_range_stack.back();
  t_range_stack.pop_back();
  if (!kernel_trace_enabled()) return;  // the trace was stopped (and the record moved out) in between
  pe->end = place_now(pe->ev.device);
}
KernelTraceScope::KernelTraceScope(const char* launch_expr) {
  if (!kernel_trace_enabled() || hostsim() || graphCaptureActive()) return;  // no timing notifiers inside a capture
  PendingEvent* pe = new_event(launcher_name(launch_expr).c_str(), 0);
  pe->ev.op = t_current_op;
  pe->start = place_now(pe->ev.device);
  rec_ = pe;
}
KernelTraceScope::~KernelTraceScope() {
  if (!rec_ || !kernel_trace_enabled()) return;
  auto* pe = static_cast<PendingEvent*>(rec_);
  pe->end = place_now(pe->ev.device);
}

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
  void mark(const char* name) const override { trace_mark(name); }
  void rangePush(const char* name) const override { trace_range_push(name); }
  void rangePop() const override { trace_range_pop(); }
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
