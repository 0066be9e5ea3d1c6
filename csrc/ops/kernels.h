// Host-side bridge from at::Tensor arguments to the device layer's C launchers.
#pragma once
#include <ATen/ATen.h>
#include <ATen/TensorIterator.h>
#include "../device/kernels_api.h"
#include "../runtime/profiler.h"
#include "common.h"

namespace catch_b200 {
namespace ops {

// Every launcher call that reaches the device is counted (benchmarks report it).
void note_kernel_launch();
long long kernel_launch_count();
void reset_kernel_launch_count();

#define B200_KERNEL_CHECK(expr)                                                                     \
  do {                                                                                              \
    ::catch_b200::ops::note_kernel_launch();                                                        \
    ::catch_b200::KernelTraceScope _trace(#expr); /* two notifiers around the launch while tracing */ \
    int _e = (expr);                                                                                \
    TORCH_CHECK(_e == 0, "b200 kernel launch failed: ", ::catch_b200::device_error_string(_e), " (", \
                #expr, ")");                                                                        \
  } while (0)

inline int to_b200_dtype(at::ScalarType t) {
  switch (t) {
    case at::kByte: return B200_U8;
    case at::kChar: return B200_I8;
    case at::kShort: return B200_I16;
    case at::kInt: return B200_I32;
    case at::kLong: return B200_I64;
    case at::kHalf: return B200_F16;
    case at::kFloat: return B200_F32;
    case at::kDouble: return B200_F64;
    case at::kBool: return B200_BOOL;
    case at::kBFloat16: return B200_BF16;
    default: TORCH_CHECK(false, "b200: unsupported dtype ", t);
  }
}

inline long long* i64ptr(const at::Tensor& t) { return reinterpret_cast<long long*>(t.data_ptr<int64_t>()); }

// Launches the element-wise family over a built TensorIterator (operand 0 is
// the output).  `s0`/`s1` are the op's scalar parameters.
void launch_ew(at::TensorIteratorBase& iter, int op, double s0, double s1, void* stream,
               std::optional<at::ScalarType> compute = std::nullopt);
// dst <- src with arbitrary strides / dtypes (same device).
void launch_copy(const at::Tensor& src, const at::Tensor& dst, void* stream);
void launch_fill(const at::Tensor& dst, double value, void* stream);

}  // namespace ops
}  // namespace catch_b200
