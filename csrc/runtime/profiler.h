// Kernel-level tracing: every launch of one of this backend's kernels can be bracketed by two notifiers and
// recorded with its name, the operator that issued it, the queue and its device time.
//
// The reference joins device kernel events to operators by correlation id with a vendor tracer
// (torch_mlu/csrc/aten/profile/profile_mlu.cpp:76-211).  Here the launch macro of the operator layer creates a
// KernelTraceScope around each launcher call while a trace is active; markers and ranges of the stock
// profiler's device stubs (mark / rangePush / rangePop) land in the same list.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace catch_b200 {

struct KernelEvent {
  std::string name;   // kernel launcher (e.g. b200_conv_fprop) or range / mark label
  std::string op;     // operator that issued it (OpScope name), empty for ranges
  int kind = 0;       // 0 kernel, 1 range, 2 mark
  int device = 0;
  uint64_t queue = 0;
  int64_t cpu_ns = 0;     // host time of the launch
  double start_us = 0;    // device time since the trace started
  double dur_us = 0;
};

bool kernel_trace_enabled();
void kernel_trace_start();
std::vector<KernelEvent> kernel_trace_stop();  // waits for the recorded work, resolves device times

// thread-local name of the operator being executed (set by OpScope)
const char* trace_current_op();
const char* trace_set_current_op(const char* name);  // returns the previous one

void trace_mark(const char* name);
void trace_range_push(const char* name);
void trace_range_pop();

class KernelTraceScope {
 public:
  explicit KernelTraceScope(const char* launch_expr);
  ~KernelTraceScope();

 private:
  void* rec_ = nullptr;
};

}  // namespace catch_b200
