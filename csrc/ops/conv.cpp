// Convolution forward / backward for the b200 device.
//
// ATen routes convolutions on an out-of-tree device to convolution_overrideable
// and convolution_backward_overrideable -- the same hook the reference used
// (torch_mlu/csrc/aten/operators/cnnl/convolution_overrideable.cpp:241-297).
// Device path: NHWC implicit-GEMM kernels on tcgen05 (conv_tcgen05.cu) for the
// dense 2-D bf16/fp16 case, a direct CUDA-core kernel for everything else
// (groups, depthwise, dilation, fp32, transposed); CPU path under host
// simulation or when the device kernel rejects the configuration.
#include "common.h"
#include "conv_impl.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

Tensor to_cpu(const Tensor& t) { return t.defined() ? t.cpu() : t; }

Tensor conv_cpu(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias, at::IntArrayRef stride,
                at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed, at::IntArrayRef output_padding,
                int64_t groups) {
  std::optional<Tensor> b;
  if (bias.has_value() && bias->defined()) b = bias->cpu();
  Tensor out = at::convolution(input.cpu(), weight.cpu(), b, stride, padding, dilation, transposed, output_padding, groups);
  return out.to(input.device());
}

std::tuple<Tensor, Tensor, Tensor> conv_backward_cpu(const Tensor& grad, const Tensor& input, const Tensor& weight,
                                                     at::IntArrayRef stride, at::IntArrayRef padding,
                                                     at::IntArrayRef dilation, bool transposed,
                                                     at::IntArrayRef output_padding, int64_t groups,
                                                     std::array<bool, 3> mask) {
  std::vector<int64_t> bias_sizes = {weight.size(transposed ? 1 : 0) * (transposed ? groups : 1)};
  auto r = at::convolution_backward(grad.cpu(), input.cpu(), weight.cpu(), bias_sizes, stride, padding, dilation,
                                    transposed, output_padding, groups, mask);
  auto mv = [&](const Tensor& t) { return t.defined() ? t.to(input.device()) : t; };
  return {mv(std::get<0>(r)), mv(std::get<1>(r)), mv(std::get<2>(r))};
}

// Memory format of a convolution result, by the stock rule: channels-last when the input or the weight is, else
// contiguous.  The kernels work channels-last, so a script that keeps everything in the default format pays one
// transposing copy per result; in exchange view() on the result behaves as it does on other devices.
bool wants_channels_last(const Tensor& input, const Tensor& weight) {
  return input.dim() == 4 && (input.suggest_memory_format() == at::MemoryFormat::ChannelsLast ||
                              weight.suggest_memory_format() == at::MemoryFormat::ChannelsLast);
}
Tensor in_format(const Tensor& t, bool channels_last) {
  if (!t.defined() || t.dim() != 4 || t.numel() == 0) return t;
  return channels_last ? t.contiguous(at::MemoryFormat::ChannelsLast) : t.contiguous();
}

Tensor convolution_overrideable(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias,
                                at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                                bool transposed, at::IntArrayRef output_padding, int64_t groups) {
  check_same_device("convolution", input, weight, bias);
  return B200_DISPATCH("convolution",
                       in_format(conv_forward_device(input, weight, bias, stride, padding, dilation, transposed, output_padding,
                                                     groups),
                                 wants_channels_last(input, weight)),
                       conv_cpu(input, weight, bias, stride, padding, dilation, transposed, output_padding, groups));
}

std::tuple<Tensor, Tensor, Tensor> convolution_backward_overrideable(
    const Tensor& grad, const Tensor& input, const Tensor& weight, at::IntArrayRef stride, at::IntArrayRef padding,
    at::IntArrayRef dilation, bool transposed, at::IntArrayRef output_padding, int64_t groups,
    std::array<bool, 3> mask) {
  auto device = [&]() {
    auto r = conv_backward_device(grad, input, weight, stride, padding, dilation, transposed, output_padding, groups, mask);
    std::get<0>(r) = in_format(std::get<0>(r), wants_channels_last(input, weight));
    return r;
  };
  return B200_DISPATCH(
      "convolution_backward", device(),
      conv_backward_cpu(grad, input, weight, stride, padding, dilation, transposed, output_padding, groups, mask));
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("convolution_overrideable", TORCH_FN(convolution_overrideable));
  m.impl("convolution_backward_overrideable", TORCH_FN(convolution_backward_overrideable));
}

}  // namespace ops
}  // namespace catch_b200
