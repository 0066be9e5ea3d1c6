// Device implementations behind the convolution operators (conv_device.cpp).
#pragma once
#include <ATen/ATen.h>
#include <array>
#include <tuple>

namespace catch_b200 {
namespace ops {

at::Tensor conv_forward_device(const at::Tensor& input, const at::Tensor& weight, const std::optional<at::Tensor>& bias,
                               at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                               bool transposed, at::IntArrayRef output_padding, int64_t groups);

std::tuple<at::Tensor, at::Tensor, at::Tensor> conv_backward_device(
    const at::Tensor& grad, const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride,
    at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed, at::IntArrayRef output_padding, int64_t groups,
    std::array<bool, 3> mask);

}  // namespace ops
}  // namespace catch_b200
