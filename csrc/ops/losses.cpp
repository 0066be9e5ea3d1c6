// Regression / binary losses composed from this backend's element-wise and reduction kernels
// (mse, smooth L1, Huber, binary cross entropy; forward and backward), so that they stay on the
// device instead of taking the CPU fallback.
//
// Parity: torch_mlu/csrc/aten/operators/cnnl/{mse_loss.cpp,smooth_l1_loss.cpp,
// binary_cross_entropy.cpp} (CNNL loss kernels with the same reduction modes).
#include <ATen/core/Reduction.h>
#include <torch/library.h>

#include "common.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

Tensor reduce(const Tensor& t, int64_t reduction) {
  if (reduction == at::Reduction::Mean) return t.mean();
  if (reduction == at::Reduction::Sum) return t.sum();
  return t;
}
// gradient of reduce(): grad_output broadcast (and divided by numel for the mean)
Tensor unreduce(const Tensor& grad_output, const Tensor& like, int64_t reduction) {
  if (reduction == at::Reduction::Mean) return grad_output / (double)like.numel();
  return grad_output;
}

Tensor mse_loss(const Tensor& self, const Tensor& target, int64_t reduction) {
  Tensor d = self - target;
  return reduce(d * d, reduction);
}
Tensor mse_loss_backward(const Tensor& grad_output, const Tensor& self, const Tensor& target, int64_t reduction) {
  return (self - target) * 2.0 * unreduce(grad_output, self, reduction);
}

Tensor smooth_l1_loss(const Tensor& self, const Tensor& target, int64_t reduction, double beta) {
  Tensor d = (self - target).abs();
  if (beta == 0.0) return reduce(d, reduction);
  Tensor quad = d * d * (0.5 / beta);
  return reduce(at::where(d.lt(beta), quad, d - 0.5 * beta), reduction);
}
Tensor smooth_l1_loss_backward(const Tensor& grad_output, const Tensor& self, const Tensor& target, int64_t reduction, double beta) {
  Tensor d = self - target;
  Tensor g = beta == 0.0 ? d.sign() : at::where(d.abs().lt(beta), d / beta, d.sign());
  return g * unreduce(grad_output, self, reduction);
}

Tensor huber_loss(const Tensor& self, const Tensor& target, int64_t reduction, double delta) {
  Tensor d = (self - target).abs();
  return reduce(at::where(d.lt(delta), d * d * 0.5, (d - 0.5 * delta) * delta), reduction);
}
Tensor huber_loss_backward(const Tensor& grad_output, const Tensor& self, const Tensor& target, int64_t reduction, double delta) {
  Tensor d = self - target;
  return at::where(d.abs().lt(delta), d, d.sign() * delta) * unreduce(grad_output, self, reduction);
}

Tensor binary_cross_entropy(const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight, int64_t reduction) {
  // log terms are clamped at -100 like the stock kernels
  Tensor l = -(target * self.log().clamp_min(-100.0) + (1.0 - target) * (1.0 - self).log().clamp_min(-100.0));
  if (weight.has_value() && weight->defined()) l = l * *weight;
  return reduce(l, reduction);
}
Tensor binary_cross_entropy_backward(const Tensor& grad_output, const Tensor& self, const Tensor& target,
                                     const std::optional<Tensor>& weight, int64_t reduction) {
  Tensor g = (self - target) / ((1.0 - self) * self).clamp_min(1e-12);
  if (weight.has_value() && weight->defined()) g = g * *weight;
  return g * unreduce(grad_output, self, reduction);
}

// log(sigmoid(x)) = min(x, 0) - log1p(exp(-|x|)); the second result is the scratch buffer of the
// CPU kernel, unused here (as in the stock GPU kernel) and returned empty.
std::tuple<Tensor, Tensor> log_sigmoid_forward(const Tensor& self) {
  Tensor out = self.clamp_max(0.0) - self.abs().neg().exp().log1p();
  return {out, at::empty({0}, self.options())};
}
Tensor log_sigmoid_backward(const Tensor& grad_output, const Tensor& self, const Tensor& buffer) {
  (void)buffer;
  return grad_output * self.neg().sigmoid();
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("mse_loss", TORCH_FN(mse_loss));
  m.impl("mse_loss_backward", TORCH_FN(mse_loss_backward));
  m.impl("smooth_l1_loss", TORCH_FN(smooth_l1_loss));
  m.impl("smooth_l1_loss_backward", TORCH_FN(smooth_l1_loss_backward));
  m.impl("huber_loss", TORCH_FN(huber_loss));
  m.impl("huber_loss_backward", TORCH_FN(huber_loss_backward));
  m.impl("binary_cross_entropy", TORCH_FN(binary_cross_entropy));
  m.impl("binary_cross_entropy_backward", TORCH_FN(binary_cross_entropy_backward));
  m.impl("log_sigmoid_forward", TORCH_FN(log_sigmoid_forward));
  m.impl("log_sigmoid_backward", TORCH_FN(log_sigmoid_backward));
}

}  // namespace ops
}  // namespace catch_b200
