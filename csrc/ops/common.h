// Shared helpers of the operator layer.
//
// Every operator wrapper follows the same steps the reference's generated
// CnnlOps layer does (torch_mlu/tools/template/cnnl_ops.cpp:38-113,
// gen.py:73-81): switch to the tensor's device, log the arguments at DEBUG
// level, optionally dump inputs, run the device kernel, on failure re-run the
// op on the CPU, optionally synchronise.  Here that is one RAII object and one
// macro instead of five generated class layers.
#pragma once
#include <ATen/ATen.h>
#include <cstdlib>
#include <ATen/native/CPUFallback.h>
#include <torch/library.h>

#include "../runtime/caching_allocator.h"
#include "../runtime/device.h"
#include "../runtime/log.h"
#include "../runtime/queue.h"
#include "../runtime/tensor_impl.h"

namespace catch_b200 {
namespace ops {

// Boxed CPU fallback used for unregistered ops and as the per-op safety net.
void cpu_fallback(const c10::OperatorHandle& op, torch::jit::Stack* stack);

// True when operators must not launch device kernels: host simulation or the
// force-CPU test mode.
inline bool use_cpu_path() { return hostsim() || flags().test_cpu_dispatch; }

// Compute kernels are registered with the dispatcher only when they can run:
// under host simulation or CATCH_B200_TEST_CPU_DISPATCH=1 (both decided when the
// library is loaded) the registrations are skipped, so every compute op reaches
// the boxed CPU fallback while factories, views and copies stay native.
// CATCH_B200_CHECK_REGISTRATIONS=1 registers them under host simulation as well: loading the library then checks
// every kernel's C++ signature against its operator schema without a GPU (calling such a kernel fails, so the
// switch is for registration checks and the operator coverage table only).
inline bool device_kernels_enabled() {
  static const bool check_only = [] {
    const char* e = std::getenv("CATCH_B200_CHECK_REGISTRATIONS");
    return e && e[0] == '1';
  }();
  return !use_cpu_path() || check_only;
}

// Sets the device of `t` current for the lifetime of the scope, logs the op
// name, and synchronises on exit when CATCH_B200_ASYNC_DISABLE is set.
class OpScope {
 public:
  OpScope(const char* name, const at::Tensor& t);
  OpScope(const char* name, int device);
  ~OpScope() noexcept(false);
  int device() const { return device_; }
  Queue queue() const { return getCurrentQueue(device_); }
  void* stream() const { return getCurrentQueue(device_).handle(); }

 private:
  const char* name_;
  const char* prev_op_ = "";
  int device_;
  DeviceSwitch sw_;
};

// Hook for the dump tool: called with the op name and its tensor arguments /
// results when dumping is active (see runtime/dumper.h).
bool dump_active();
void dump_op_begin(const char* name);
void dump_tensor(const char* label, const at::Tensor& t);
void dump_op_end();

std::string describe(const at::Tensor& t);  // "Float[2, 3]{strides}@b200:0"

// Workspace from the caching allocator, freed (stream-ordered) on scope exit.
class Workspace {
 public:
  Workspace(size_t bytes, const OpScope& s) : ptr_(bytes ? raw_alloc(bytes, s.device(), s.queue()) : nullptr) {}
  ~Workspace() {
    if (ptr_) raw_free(ptr_);
  }
  void* get() const { return ptr_; }
  template <typename T>
  T* as() const { return static_cast<T*>(ptr_); }

 private:
  void* ptr_;
};

// Runs `device_expr`; when it throws and per-op try/catch is enabled, logs the
// failure and evaluates `cpu_expr` instead (reference: ENABLE_CNNL_TRYCATCH).
#define B200_DISPATCH(opname, device_expr, cpu_expr)                                        \
  [&]() {                                                                                   \
    if (::catch_b200::ops::use_cpu_path()) return cpu_expr;                                 \
    if (!::catch_b200::flags().op_trycatch) return device_expr;                             \
    try {                                                                                   \
      return device_expr;                                                                   \
    } catch (const c10::OutOfMemoryError&) {                                                \
      throw;                                                                                \
    } catch (const std::exception& e) {                                                     \
      B200LOG(WARNING) << opname << " failed on the device (" << e.what()                   \
                       << "); running it on the CPU instead.";                              \
      return cpu_expr;                                                                      \
    }                                                                                       \
  }()

// Raises, in the words of the stock backends, when an argument lives on another device than the first one: a kernel
// handed a host pointer (or another device's) would otherwise read memory it must not.  Undefined / absent tensors pass.
inline void same_device_one(const char* op, const at::Tensor& first, const at::Tensor& t) {
  if (!t.defined()) return;
  TORCH_CHECK(t.device() == first.device(), "Expected all tensors to be on the same device, but found at least two devices, ",
              first.device(), " and ", t.device(), "! (when checking the arguments of ", op, ")");
}
inline void same_device_one(const char* op, const at::Tensor& first, const std::optional<at::Tensor>& t) {
  if (t.has_value()) same_device_one(op, first, *t);
}
template <typename... Ts>
inline void check_same_device(const char* op, const at::Tensor& first, const Ts&... rest) {
  (same_device_one(op, first, rest), ...);
}

// Calls the boxed CPU fallback for one ATen overload with unboxed arguments,
// e.g. B200_CPU(add_Tensor, self, other, alpha).
#define B200_CPU(OP, ...) \
  at::native::call_fallback_fn<&::catch_b200::ops::cpu_fallback, at::_ops::OP>::call(__VA_ARGS__)
#define B200_CPU_SYMINT(OP, ...) \
  at::native::call_fallback_fn_symint<&::catch_b200::ops::cpu_fallback, at::_ops::OP>::call(__VA_ARGS__)

}  // namespace ops
}  // namespace catch_b200
