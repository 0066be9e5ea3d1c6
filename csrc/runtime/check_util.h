// Small checking helpers shared by C++ tests and operator wrappers.
//
// * assertTensorsEqual: the comparison the reference's C++ tests use
//   (torch_mlu/csrc/aten/util/assert_tensor.cpp:48-105): maximum absolute error by default, or one of
//   three relative measures.  Throws c10::Error with the measured value in the message.
// * batchCheckErrors: reports the LAPACK-style `info` codes of a batched factorisation
//   (torch_mlu/csrc/aten/util/matrix_util.cpp:38-61).  Returns the number of failed batches.
#pragma once
#include <ATen/ATen.h>

namespace catch_b200 {

struct TensorDiff {
  double max_abs = 0;    // max |a - b|
  double rel_rms = 0;    // sqrt(sum (a-b)^2 / sum a^2)            (use_MSE)
  double rel_abs = 0;    // sum |a-b| / sum |a|                     (use_RAE)
  double rel_mean = 0;   // (mean|a| - mean|b|) / mean|a|           (use_RMA)
};
TensorDiff tensorDiff(const at::Tensor& a, const at::Tensor& b);

void assertTensorsEqual(const at::Tensor& a, const at::Tensor& b, double prec = 0.0, bool use_MSE = false,
                        bool use_RAE = false, bool use_RMA = false);

int64_t batchCheckErrors(const at::Tensor& infos, const char* name, bool allow_singular = false);

}  // namespace catch_b200
