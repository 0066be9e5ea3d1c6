// softmax / log_softmax (+ backward), nll_loss (+ backward) and the fused
// softmax-cross-entropy custom op.
//
// Parity: torch_mlu/csrc/aten/operators/cnnl/softmax.cpp:91, nllloss.cpp:148,
// nllloss_backward.cpp:137 (half inputs are computed in fp32 there as here).
#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

bool f_ok(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf; }

// move `dim` last and make rows contiguous; returns the permuted dense tensor
Tensor rows_last(const Tensor& x, int64_t dim) {
  if (dim == x.dim() - 1) return x.contiguous();
  return x.transpose(dim, -1).contiguous();
}
Tensor restore(const Tensor& y, int64_t dim, int64_t ndim) {
  if (dim == ndim - 1) return y;
  return y.transpose(dim, -1).contiguous();  // a contiguous result, as from the stock kernels (callers may view() it)
}

Tensor softmax_impl(const Tensor& self, int64_t dim, bool half_to_float, int log_mode) {
  TORCH_CHECK(f_ok(self.scalar_type()), "b200 softmax: unsupported dtype ", self.scalar_type());
  OpScope scope(log_mode ? "_log_softmax" : "_softmax", self);
  if (self.dim() == 0) {
    Tensor o = at::empty_like(self, self.options().dtype(half_to_float ? at::kFloat : self.scalar_type()));
    return o.fill_(log_mode ? 0.0 : 1.0);
  }
  dim = at::maybe_wrap_dim(dim, self.dim());
  Tensor x = rows_last(self, dim);
  const at::ScalarType odt = half_to_float ? at::kFloat : self.scalar_type();
  Tensor y = at::empty_like(x, x.options().dtype(odt));
  const int64_t cols = x.size(-1), rows = cols ? x.numel() / cols : 0;
  B200_KERNEL_CHECK(b200_softmax_fwd(x.data_ptr(), to_b200_dtype(x.scalar_type()), y.data_ptr(), to_b200_dtype(odt), rows,
                                     (int)cols, log_mode, scope.stream()));
  return restore(y, dim, self.dim());
}
Tensor softmax_bwd_impl(const Tensor& grad, const Tensor& output, int64_t dim, at::ScalarType input_dtype, int log_mode) {
  TORCH_CHECK(f_ok(grad.scalar_type()) && grad.scalar_type() == output.scalar_type(), "b200 softmax_backward: unsupported dtypes");
  OpScope scope(log_mode ? "_log_softmax_backward_data" : "_softmax_backward_data", grad);
  dim = at::maybe_wrap_dim(dim, grad.dim());
  if (grad.dim() == 0) return at::zeros_like(grad, grad.options().dtype(input_dtype));
  Tensor g = rows_last(grad, dim), y = rows_last(output, dim);
  Tensor dx = at::empty_like(g, g.options().dtype(input_dtype));
  const int64_t cols = g.size(-1), rows = cols ? g.numel() / cols : 0;
  B200_KERNEL_CHECK(b200_softmax_bwd(g.data_ptr(), y.data_ptr(), to_b200_dtype(g.scalar_type()), dx.data_ptr(),
                                     to_b200_dtype(input_dtype), rows, (int)cols, log_mode, scope.stream()));
  return restore(dx, dim, grad.dim());
}

Tensor k_softmax(const Tensor& self, int64_t dim, bool h2f) {
  return B200_DISPATCH("_softmax", softmax_impl(self, dim, h2f, 0), B200_CPU(_softmax, self, dim, h2f));
}
Tensor k_log_softmax(const Tensor& self, int64_t dim, bool h2f) {
  return B200_DISPATCH("_log_softmax", softmax_impl(self, dim, h2f, 1), B200_CPU(_log_softmax, self, dim, h2f));
}
Tensor k_softmax_backward(const Tensor& grad, const Tensor& output, int64_t dim, at::ScalarType idt) {
  return B200_DISPATCH("_softmax_backward_data", softmax_bwd_impl(grad, output, dim, idt, 0),
                       B200_CPU(_softmax_backward_data, grad, output, dim, idt));
}
Tensor k_log_softmax_backward(const Tensor& grad, const Tensor& output, int64_t dim, at::ScalarType idt) {
  return B200_DISPATCH("_log_softmax_backward_data", softmax_bwd_impl(grad, output, dim, idt, 1),
                       B200_CPU(_log_softmax_backward_data, grad, output, dim, idt));
}

std::tuple<Tensor, Tensor> nll_fwd_device(const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight,
                                          int64_t reduction, int64_t ignore_index) {
  TORCH_CHECK(f_ok(self.scalar_type()) && self.dim() >= 1 && self.dim() <= 2 && target.scalar_type() == at::kLong,
              "b200 nll_loss: unsupported arguments");
  OpScope scope("nll_loss_forward", self);
  Tensor x = self.dim() == 1 ? self.unsqueeze(0).contiguous() : self.contiguous();
  Tensor t = target.dim() == 0 ? target.unsqueeze(0).contiguous() : target.contiguous();
  const int64_t rows = x.size(0), cols = x.size(1);
  TORCH_CHECK(t.numel() == rows, "nll_loss: target size mismatch");
  Tensor w;
  const void* wp = nullptr;
  if (weight.has_value() && weight->defined()) {
    w = weight->to(self.scalar_type()).contiguous();
    wp = w.data_ptr();
  }
  Tensor out = reduction == 0 ? at::empty({rows}, self.options()) : at::empty({}, self.options());
  if (reduction == 0 && self.dim() == 1) out = at::empty({}, self.options());
  Tensor total = at::empty({}, self.options());
  B200_KERNEL_CHECK(b200_nll_loss_fwd(x.data_ptr(), to_b200_dtype(x.scalar_type()), i64ptr(t), wp, rows,
                                      (int)cols, (int)reduction, ignore_index, out.data_ptr(), total.data_ptr(),
                                      scope.stream()));
  return {out, total};
}
std::tuple<Tensor, Tensor> k_nll_loss_forward(const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight,
                                              int64_t reduction, c10::SymInt ignore_index) {
  const int64_t ig = ignore_index.expect_int();
  check_same_device("nll_loss", self, target, weight);
  return B200_DISPATCH("nll_loss_forward", nll_fwd_device(self, target, weight, reduction, ig),
                       B200_CPU_SYMINT(nll_loss_forward, self, target, weight, reduction, ignore_index));
}
Tensor nll_bwd_device(const Tensor& grad, const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight,
                      int64_t reduction, int64_t ignore_index, const Tensor& total_weight) {
  TORCH_CHECK(f_ok(self.scalar_type()) && self.dim() >= 1 && self.dim() <= 2, "b200 nll_loss_backward: unsupported arguments");
  OpScope scope("nll_loss_backward", self);
  Tensor gi = at::zeros_like(self, at::MemoryFormat::Contiguous);
  const int64_t rows = self.dim() == 1 ? 1 : self.size(0), cols = self.size(-1);
  Tensor t = target.contiguous();
  Tensor g = grad.to(self.scalar_type()).contiguous();
  Tensor tw = total_weight.to(self.scalar_type());
  Tensor w;
  const void* wp = nullptr;
  if (weight.has_value() && weight->defined()) {
    w = weight->to(self.scalar_type()).contiguous();
    wp = w.data_ptr();
  }
  B200_KERNEL_CHECK(b200_nll_loss_bwd(g.data_ptr(), to_b200_dtype(self.scalar_type()), i64ptr(t), wp,
                                      tw.data_ptr(), rows, (int)cols, (int)reduction, ignore_index, gi.data_ptr(),
                                      scope.stream()));
  return gi;
}
Tensor k_nll_loss_backward(const Tensor& grad, const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight,
                           int64_t reduction, c10::SymInt ignore_index, const Tensor& total_weight) {
  const int64_t ig = ignore_index.expect_int();
  return B200_DISPATCH("nll_loss_backward", nll_bwd_device(grad, self, target, weight, reduction, ig, total_weight),
                       B200_CPU_SYMINT(nll_loss_backward, grad, self, target, weight, reduction, ignore_index, total_weight));
}

}  // namespace

// Fused softmax + cross entropy (mean over non-ignored rows).  Returns (loss, dlogits)
// where dlogits already is d(loss)/d(logits); the Python autograd wrapper multiplies
// by the incoming gradient.
std::tuple<at::Tensor, at::Tensor> softmax_cross_entropy(const at::Tensor& logits, const at::Tensor& target,
                                                         int64_t ignore_index, double label_smoothing) {
  check_same_device("softmax_cross_entropy", logits, target);
  TORCH_CHECK(logits.dim() == 2 && target.dim() == 1 && target.scalar_type() == at::kLong, "softmax_cross_entropy: logits [N, C], target [N] int64");
  if (use_cpu_path() || !f_ok(logits.scalar_type())) {
    at::Tensor x = logits.detach().to(at::kFloat);
    at::Tensor loss = at::cross_entropy_loss(x, target, {}, at::Reduction::Mean, ignore_index, label_smoothing);
    const int64_t C = x.size(1);
    at::Tensor valid = target.ne(ignore_index);
    at::Tensor safe_t = at::where(valid, target, at::zeros_like(target));
    at::Tensor tgt = at::one_hot(safe_t.cpu(), C).to(x.device()).to(at::kFloat) * (1.0 - label_smoothing) + label_smoothing / C;
    at::Tensor g = (at::softmax(x, 1) - tgt) * valid.to(at::kFloat).unsqueeze(1) / valid.sum().clamp_min(1).to(at::kFloat);
    return {loss.detach(), g.to(logits.scalar_type())};
  }
  OpScope scope("softmax_cross_entropy", logits);
  at::Tensor x = logits.contiguous(), t = target.contiguous();
  const int64_t rows = x.size(0), cols = x.size(1);
  auto fopt = logits.options().dtype(at::kFloat);
  at::Tensor row_loss = at::empty({rows}, fopt), n_valid = at::empty({1}, fopt);
  at::Tensor dl = at::empty_like(x);
  B200_KERNEL_CHECK(b200_softmax_xent(x.data_ptr(), to_b200_dtype(x.scalar_type()), i64ptr(t), rows, (int)cols,
                                      ignore_index, (float)label_smoothing, row_loss.data_ptr<float>(),
                                      n_valid.data_ptr<float>(), dl.data_ptr(), to_b200_dtype(x.scalar_type()), 1.0f,
                                      scope.stream()));
  at::Tensor loss = row_loss.sum() / n_valid.squeeze(0).clamp_min(1.0);
  return {loss, dl};
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("_softmax", TORCH_FN(k_softmax));
  m.impl("_log_softmax", TORCH_FN(k_log_softmax));
  m.impl("_softmax_backward_data", TORCH_FN(k_softmax_backward));
  m.impl("_log_softmax_backward_data", TORCH_FN(k_log_softmax_backward));
  m.impl("nll_loss_forward", TORCH_FN(k_nll_loss_forward));
  m.impl("nll_loss_backward", TORCH_FN(k_nll_loss_backward));
}

}  // namespace ops
}  // namespace catch_b200
