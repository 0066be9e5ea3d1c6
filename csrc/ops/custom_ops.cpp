// Custom operator schemas of the backend (namespace catch_b200):
//   conv_bn_act / linear_act        -- fused inference ops produced by the fusion pass
//   conv2d / linear (quantized)     -- int8 ops with the reference's argument order
//                                      (torch_mlu/core/quantized/modules/conv.py:182-190, linear.py:44-48)
//   softmax_cross_entropy           -- fused loss (value and logits gradient)
//   fused_sgd_step / fused_adamw_step
//   dump                            -- device printf of a tensor (reference: torch_mlu::dump)
#include <torch/library.h>
#include "common.h"

namespace catch_b200 {
namespace ops {

at::Tensor linear_act(const at::Tensor& x, const at::Tensor& w, const std::optional<at::Tensor>& bias, int64_t act);
at::Tensor conv_bn_act_device(const at::Tensor& input, const at::Tensor& weight, const std::optional<at::Tensor>& scale,
                              const std::optional<at::Tensor>& bias, const std::optional<at::Tensor>& residual,
                              at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups,
                              int64_t act);
std::tuple<at::Tensor, at::Tensor> softmax_cross_entropy(const at::Tensor& logits, const at::Tensor& target,
                                                         int64_t ignore_index, double label_smoothing);
void fused_sgd_step(at::TensorList params, at::TensorList grads, at::TensorList momentum_bufs, at::TensorList lowp,
                    double lr, double momentum, double dampening, double weight_decay, bool nesterov, bool first_step,
                    double grad_scale);
void fused_adamw_step(at::TensorList params, at::TensorList grads, at::TensorList exp_avg, at::TensorList exp_avg_sq,
                      at::TensorList lowp, double lr, double beta1, double beta2, double eps, double weight_decay,
                      int64_t step, double grad_scale, bool adam_l2_mode);
bool dump_tensor_device(const at::Tensor& t);
std::tuple<at::Tensor, at::Tensor, at::Tensor> batch_norm_act(const at::Tensor& input, const std::optional<at::Tensor>& weight,
                                                              const std::optional<at::Tensor>& bias,
                                                              const std::optional<at::Tensor>& running_mean,
                                                              const std::optional<at::Tensor>& running_var,
                                                              const std::optional<at::Tensor>& residual, bool training,
                                                              double momentum, double eps, int64_t act,
                                                              const std::optional<at::Tensor>& channel_sums);
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> batch_norm_act_mask(
    const at::Tensor& input, const std::optional<at::Tensor>& weight, const std::optional<at::Tensor>& bias,
    const std::optional<at::Tensor>& running_mean, const std::optional<at::Tensor>& running_var,
    const std::optional<at::Tensor>& residual, bool training, double momentum, double eps, int64_t act,
    const std::optional<at::Tensor>& channel_sums, const std::optional<at::Tensor>& num_batches_tracked);
std::tuple<at::Tensor, at::Tensor> conv_backward_fp32w_device(const at::Tensor& grad, const at::Tensor& input,
                                                              const at::Tensor& weight, at::IntArrayRef stride,
                                                              at::IntArrayRef padding, bool need_dx, bool need_dw,
                                                              const std::optional<at::Tensor>& accum,
                                                              const std::optional<at::Tensor>& dx_add);
std::tuple<at::Tensor, at::Tensor> conv_stats_device(const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride,
                                                     at::IntArrayRef padding);
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> dropout_add_layer_norm(
    const at::Tensor& h, const at::Tensor& residual, const std::optional<at::Tensor>& weight, const std::optional<at::Tensor>& bias,
    double p, bool training, double eps);
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> dropout_add_layer_norm_backward(
    const at::Tensor& dy, const at::Tensor& s, const at::Tensor& mask, const std::optional<at::Tensor>& weight,
    const at::Tensor& mean, const at::Tensor& rstd, double p);
at::Tensor gemm_nd(const at::Tensor& a, const at::Tensor& b, const std::optional<at::Tensor>& out, double alpha);
std::tuple<at::Tensor, at::Tensor, at::Tensor> linear_backward_fp32w(const at::Tensor& grad, const at::Tensor& x, const at::Tensor& w,
                                                                     bool need_dx, bool need_dw, bool need_db,
                                                                     const std::optional<at::Tensor>& accum_w,
                                                                     const std::optional<at::Tensor>& accum_b);
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> batch_norm_act_backward(
    const at::Tensor& grad_out, const at::Tensor& out, const at::Tensor& input, const std::optional<at::Tensor>& weight,
    const std::optional<at::Tensor>& running_mean, const at::Tensor& save_mean, const at::Tensor& save_invstd, bool training,
    int64_t act, bool has_residual);

// act(conv(x, w) * scale + bias + residual); runs the fused tcgen05 kernel when it
// can, otherwise composes stock ops (which themselves dispatch to this backend).
static at::Tensor conv_bn_act(const at::Tensor& input, const at::Tensor& weight, const std::optional<at::Tensor>& scale,
                              const std::optional<at::Tensor>& bias, const std::optional<at::Tensor>& residual,
                              at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups,
                              int64_t act) {
  check_same_device("conv_bn_act", input, weight, scale, bias, residual);
  auto compose = [&]() {
    at::Tensor y = at::conv2d(input, weight, {}, stride, padding, dilation, groups);
    if (scale.has_value() && scale->defined()) y = y * scale->to(y.scalar_type()).view({1, -1, 1, 1});
    if (bias.has_value() && bias->defined()) y = y + bias->to(y.scalar_type()).view({1, -1, 1, 1});
    if (residual.has_value() && residual->defined()) y = y + *residual;
    if (act == 1) y = at::relu(y);
    return y;
  };
  if (use_cpu_path() || !is_b200(input)) return compose();
  if (!flags().op_trycatch)
    return conv_bn_act_device(input, weight, scale, bias, residual, stride, padding, dilation, groups, act);
  try {
    return conv_bn_act_device(input, weight, scale, bias, residual, stride, padding, dilation, groups, act);
  } catch (const c10::OutOfMemoryError&) {
    throw;
  } catch (const std::exception& e) {
    B200LOG(DBG) << "conv_bn_act: fused kernel rejected the configuration (" << e.what() << "); composing stock ops.";
    return compose();
  }
}

TORCH_LIBRARY(catch_b200, m) {
  m.def("conv_bn_act(Tensor input, Tensor weight, Tensor? scale, Tensor? bias, Tensor? residual, int[] stride, "
        "int[] padding, int[] dilation, int groups, int act) -> Tensor");
  m.def("linear_act(Tensor input, Tensor weight, Tensor? bias, int act) -> Tensor");
  m.def("softmax_cross_entropy(Tensor logits, Tensor target, int ignore_index, float label_smoothing) -> (Tensor, Tensor)");
  m.def("fused_sgd_step(Tensor[] params, Tensor[] grads, Tensor[] momentum_bufs, Tensor[] lowp, float lr, float momentum, "
        "float dampening, float weight_decay, bool nesterov, bool first_step, float grad_scale) -> ()");
  m.def("fused_adamw_step(Tensor[] params, Tensor[] grads, Tensor[] exp_avg, Tensor[] exp_avg_sq, Tensor[] lowp, float lr, "
        "float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale, bool adam_l2_mode) -> ()");
  m.def("dump(Tensor t) -> bool");
  m.def("batch_norm_act(Tensor input, Tensor? weight, Tensor? bias, Tensor(a!)? running_mean, Tensor(b!)? running_var, "
        "Tensor? residual, bool training, float momentum, float eps, int act, Tensor? channel_sums=None) -> (Tensor, Tensor, Tensor)");
  // like batch_norm_act; the 4th result is a bit mask of the positive outputs (empty if not produced) that
  // batch_norm_act_backward accepts in place of `out`; num_batches_tracked (int64, optional) is incremented
  m.def("batch_norm_act_mask(Tensor input, Tensor? weight, Tensor? bias, Tensor(a!)? running_mean, Tensor(b!)? running_var, "
        "Tensor? residual, bool training, float momentum, float eps, int act, Tensor? channel_sums=None, "
        "Tensor(c!)? num_batches_tracked=None) -> (Tensor, Tensor, Tensor, Tensor)");
  // convolution (no bias, 16-bit) that also returns fp64 [2 * Cout] channel sums / sums of squares of its output
  m.def("conv2d_stats(Tensor input, Tensor weight, int[] stride, int[] padding) -> (Tensor, Tensor)");
  // (grad_input, grad_weight) of a dense 16-bit convolution; grad_weight is fp32 (undefined results where not
  // needed).  With `accum` (flat fp32, memory order [K][R][S][C]) the weight gradient is added into it in place.
  // dx_add: another gradient of `input` (a skip connection's) that the data-gradient epilogue adds to grad_input.
  m.def("conv2d_backward_fp32w(Tensor grad, Tensor input, Tensor weight, int[] stride, int[] padding, bool need_dx, "
        "bool need_dw, Tensor(a!)? accum=None, Tensor? dx_add=None) -> (Tensor, Tensor)");
  // backward of a 16-bit linear layer with fp32 master weights: (grad_input, grad_weight fp32, grad_bias fp32); with
  // accum_w / accum_b the parameter gradients are added into those flat fp32 buffers and not returned
  m.def("linear_backward_fp32w(Tensor grad, Tensor input, Tensor weight, bool need_dx, bool need_dw, bool need_db, "
        "Tensor(a!)? accum_w=None, Tensor(b!)? accum_b=None) -> (Tensor, Tensor, Tensor)");
  // alpha * a @ b over 4-D operands [B1, B2, M, K] x [B1, B2, K, N] with arbitrary batch strides (no head-split copies);
  // `out` may be a strided [B1, B2, M, N] view
  m.def("gemm_nd(Tensor a, Tensor b, Tensor(a!)? out=None, float alpha=1.0) -> Tensor");
  // s = residual + dropout(h); y = layer_norm(s): (y, s, mask, mean, rstd), one kernel; and its backward (ds, dh, dgamma, dbeta)
  m.def("dropout_add_layer_norm(Tensor h, Tensor residual, Tensor? weight, Tensor? bias, float p, bool training, float eps) -> "
        "(Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("dropout_add_layer_norm_backward(Tensor dy, Tensor s, Tensor mask, Tensor? weight, Tensor mean, Tensor rstd, float p) -> "
        "(Tensor, Tensor, Tensor, Tensor)");
  m.def("batch_norm_act_backward(Tensor grad_out, Tensor out, Tensor input, Tensor? weight, Tensor? running_mean, "
        "Tensor save_mean, Tensor save_invstd, bool training, int act, bool has_residual) -> (Tensor, Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(catch_b200, CompositeExplicitAutograd, m) {
  m.impl("conv_bn_act", TORCH_FN(conv_bn_act));
  m.impl("linear_act", TORCH_FN(linear_act));
  m.impl("softmax_cross_entropy", TORCH_FN(softmax_cross_entropy));
  m.impl("fused_sgd_step", TORCH_FN(fused_sgd_step));
  m.impl("fused_adamw_step", TORCH_FN(fused_adamw_step));
  m.impl("dump", TORCH_FN(dump_tensor_device));
  m.impl("batch_norm_act", TORCH_FN(batch_norm_act));
  m.impl("conv2d_stats", TORCH_FN(conv_stats_device));
  m.impl("conv2d_backward_fp32w", TORCH_FN(conv_backward_fp32w_device));
  m.impl("batch_norm_act_mask", TORCH_FN(batch_norm_act_mask));
  m.impl("linear_backward_fp32w", TORCH_FN(linear_backward_fp32w));
  m.impl("gemm_nd", TORCH_FN(gemm_nd));
  m.impl("dropout_add_layer_norm", TORCH_FN(dropout_add_layer_norm));
  m.impl("dropout_add_layer_norm_backward", TORCH_FN(dropout_add_layer_norm_backward));
  m.impl("batch_norm_act_backward", TORCH_FN(batch_norm_act_backward));
}

}  // namespace ops
}  // namespace catch_b200
