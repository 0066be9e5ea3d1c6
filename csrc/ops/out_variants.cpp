// out= (and a few in-place) overloads of operators whose functional form has a device kernel: the result is
// computed by that kernel and moved into the caller's tensor (resized as PyTorch's out= contract asks).
// The reference registers the same overloads one by one (torch_mlu/tools/mlu_functions.yaml: gather.out,
// index_select.out, topk.values, max.dim_max, sum.IntList_out, ...).
#include <ATen/ATen.h>
#include <torch/library.h>

#include "common.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

Tensor& assign(Tensor& out, const Tensor& value) {
  if (out.sizes() != value.sizes()) out.resize_(value.sizes());
  out.copy_(value);
  return out;
}

Tensor& adaptive_avg_pool2d_out(const Tensor& self, c10::SymIntArrayRef size, Tensor& out) {
  return assign(out, at::_adaptive_avg_pool2d_symint(self, size));
}
std::tuple<Tensor&, Tensor&> adaptive_max_pool2d_out(const Tensor& self, at::IntArrayRef size, Tensor& out, Tensor& indices) {
  auto r = at::adaptive_max_pool2d(self, size);
  assign(out, std::get<0>(r));
  assign(indices, std::get<1>(r));
  return {out, indices};
}
Tensor& adaptive_max_pool2d_backward_out(const Tensor& grad, const Tensor& self, const Tensor& indices, Tensor& grad_input) {
  return assign(grad_input, at::adaptive_max_pool2d_backward(grad, self, indices));
}
Tensor& all_out(const Tensor& self, int64_t dim, bool keepdim, Tensor& out) { return assign(out, at::all(self, dim, keepdim)); }
Tensor& bce_out(const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight, int64_t reduction, Tensor& out) {
  return assign(out, at::binary_cross_entropy(self, target, weight, reduction));
}
Tensor& bce_backward_out(const Tensor& grad, const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight,
                         int64_t reduction, Tensor& grad_input) {
  return assign(grad_input, at::binary_cross_entropy_backward(grad, self, target, weight, reduction));
}
Tensor& clamp_min_out(const Tensor& self, const at::Scalar& min, Tensor& out) { return assign(out, at::clamp_min(self, min)); }
Tensor& gather_out(const Tensor& self, int64_t dim, const Tensor& index, bool sparse_grad, Tensor& out) {
  return assign(out, at::gather(self, dim, index, sparse_grad));
}
Tensor& index_select_out(const Tensor& self, int64_t dim, const Tensor& index, Tensor& out) {
  return assign(out, at::index_select(self, dim, index));
}
Tensor& leaky_relu_out(const Tensor& self, const at::Scalar& slope, Tensor& out) { return assign(out, at::leaky_relu(self, slope)); }
Tensor& masked_select_out(const Tensor& self, const Tensor& mask, Tensor& out) { return assign(out, at::masked_select(self, mask)); }
std::tuple<Tensor&, Tensor&> max_dim_out(const Tensor& self, int64_t dim, bool keepdim, Tensor& values, Tensor& indices) {
  auto r = at::max(self, dim, keepdim);
  assign(values, std::get<0>(r));
  assign(indices, std::get<1>(r));
  return {values, indices};
}
Tensor& mean_out(const Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype, Tensor& out) {
  return assign(out, at::mean(self, dim, keepdim, dtype));
}
Tensor& nonzero_out(const Tensor& self, Tensor& out) { return assign(out, at::nonzero(self)); }
Tensor& pow_scalar_(Tensor& self, const at::Scalar& exponent) { return assign(self, at::pow(self, exponent)); }
Tensor& prod_int_out(const Tensor& self, int64_t dim, bool keepdim, std::optional<at::ScalarType> dtype, Tensor& out) {
  return assign(out, at::prod(self, dim, keepdim, dtype));
}
Tensor& smooth_l1_out(const Tensor& self, const Tensor& target, int64_t reduction, double beta, Tensor& out) {
  return assign(out, at::smooth_l1_loss(self, target, reduction, beta));
}
Tensor& smooth_l1_backward_out(const Tensor& grad, const Tensor& self, const Tensor& target, int64_t reduction, double beta,
                               Tensor& grad_input) {
  return assign(grad_input, at::smooth_l1_loss_backward(grad, self, target, reduction, beta));
}
Tensor& sum_out(const Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype, Tensor& out) {
  return assign(out, at::sum(self, dim, keepdim, dtype));
}
Tensor& threshold_out(const Tensor& self, const at::Scalar& threshold, const at::Scalar& value, Tensor& out) {
  return assign(out, at::threshold(self, threshold, value));
}
std::tuple<Tensor&, Tensor&> topk_out(const Tensor& self, c10::SymInt k, int64_t dim, bool largest, bool sorted, Tensor& values,
                                      Tensor& indices) {
  auto r = at::topk_symint(self, k, dim, largest, sorted);
  assign(values, std::get<0>(r));
  assign(indices, std::get<1>(r));
  return {values, indices};
}
Tensor& upsample_bilinear2d_out(const Tensor& self, c10::SymIntArrayRef size, bool align_corners, std::optional<double> sh,
                                std::optional<double> sw, Tensor& out) {
  return assign(out, at::upsample_bilinear2d_symint(self, size, align_corners, sh, sw));
}
Tensor& upsample_nearest2d_out(const Tensor& self, c10::SymIntArrayRef size, std::optional<double> sh, std::optional<double> sw,
                               Tensor& out) {
  return assign(out, at::upsample_nearest2d_symint(self, size, sh, sw));
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("adaptive_avg_pool2d.out", TORCH_FN(adaptive_avg_pool2d_out));
  m.impl("adaptive_max_pool2d.out", TORCH_FN(adaptive_max_pool2d_out));
  m.impl("adaptive_max_pool2d_backward.grad_input", TORCH_FN(adaptive_max_pool2d_backward_out));
  m.impl("all.out", TORCH_FN(all_out));
  m.impl("binary_cross_entropy.out", TORCH_FN(bce_out));
  m.impl("binary_cross_entropy_backward.grad_input", TORCH_FN(bce_backward_out));
  m.impl("clamp_min.out", TORCH_FN(clamp_min_out));
  m.impl("gather.out", TORCH_FN(gather_out));
  m.impl("index_select.out", TORCH_FN(index_select_out));
  m.impl("leaky_relu.out", TORCH_FN(leaky_relu_out));
  m.impl("masked_select.out", TORCH_FN(masked_select_out));
  m.impl("max.dim_max", TORCH_FN(max_dim_out));
  m.impl("mean.out", TORCH_FN(mean_out));
  m.impl("nonzero.out", TORCH_FN(nonzero_out));
  m.impl("pow_.Scalar", TORCH_FN(pow_scalar_));
  m.impl("prod.int_out", TORCH_FN(prod_int_out));
  m.impl("smooth_l1_loss.out", TORCH_FN(smooth_l1_out));
  m.impl("smooth_l1_loss_backward.grad_input", TORCH_FN(smooth_l1_backward_out));
  m.impl("sum.IntList_out", TORCH_FN(sum_out));
  m.impl("threshold.out", TORCH_FN(threshold_out));
  m.impl("topk.values", TORCH_FN(topk_out));
  m.impl("upsample_bilinear2d.out", TORCH_FN(upsample_bilinear2d_out));
  m.impl("upsample_nearest2d.out", TORCH_FN(upsample_nearest2d_out));
}

}  // namespace ops
}  // namespace catch_b200
