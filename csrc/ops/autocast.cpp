// Autocast policies for the b200 device (dispatch key AutocastPrivateUse1):
// matmul / convolution class ops run in the autocast dtype (bf16 or fp16),
// numerically sensitive ops in fp32, mixed-input ops promote.  The op lists are
// PyTorch's shared policy lists, so behaviour matches the stock CUDA autocast.
// The reference has no mixed-precision training at all
// (docs/user_guide/source/pytorch_8_training/Pytorch_training.rst:24).
#include <ATen/autocast_mode.h>
#include <torch/library.h>

namespace {
using namespace at::autocast;
using at::DimnameList;
using at::IntArrayRef;
using at::Scalar;
using at::ScalarType;
using at::Tensor;

#define B200_LOWP(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, lower_precision_fp)
#define B200_FP32(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, fp32)
#define B200_PROMOTE(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, promote)
// reductions and softmax with an optional dtype argument: fp32 output unless the caller asked for a dtype
#define B200_FP32_OPT_DTYPE(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, fp32_set_opt_dtype)

TORCH_LIBRARY_IMPL(_, AutocastPrivateUse1, m) { m.fallback(torch::CppFunction::makeFallthrough()); }

TORCH_LIBRARY_IMPL(aten, AutocastPrivateUse1, m) {
  AT_FORALL_LOWER_PRECISION_FP(B200_LOWP)
  AT_FORALL_FP32(B200_FP32)
  AT_FORALL_PROMOTE(B200_PROMOTE)
  AT_FORALL_FP32_SET_OPT_DTYPE(B200_FP32_OPT_DTYPE)
  AT_FORALL_DIFFERENT_REDISPATCH_SIGNATURE(KERNEL_DIFFERENT_REDISPATCH_SIGNATURE_PRIVATEUSEONE)
}
}  // namespace
