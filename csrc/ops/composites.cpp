// Operators without a kernel of their own that are built from this backend's device kernels instead of taking the
// boxed CPU fallback (two copies over PCIe and a host computation per call): var / std (+ _mean forms), dot, addmv,
// flip, roll, elu_backward, hardswish_backward, logit, xlogy, the group-norm gradient and the LSTM / GRU cells.  The reference runs the same set through its
// kernel library (torch_mlu/csrc/aten/operators/cnnl/{std.cpp,var.cpp,dot.cpp,addmv.cpp,flip.cpp,roll.cpp}).
// Every piece below is a device operator of this backend (reductions, element-wise kernels, index_select, GEMM), so
// the data never leaves the device; accumulation happens in fp32 for 16-bit inputs.
#include <numeric>

#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Scalar;
using at::Tensor;

bool is_float_dtype(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf; }

// ---- var / std -----------------------------------------------------------------------------------------
std::vector<int64_t> reduce_dims(const Tensor& self, at::OptionalIntArrayRef dim) {
  std::vector<int64_t> dims;
  if (dim.has_value() && !dim->empty()) {
    for (int64_t d : *dim) dims.push_back(at::maybe_wrap_dim(d, self.dim()));
  } else {
    dims.resize(self.dim());
    std::iota(dims.begin(), dims.end(), 0);
  }
  return dims;
}

// (variance or standard deviation, mean) with the reduced dimensions kept or dropped
std::pair<Tensor, Tensor> var_mean_device(const Tensor& self, at::OptionalIntArrayRef dim, const std::optional<Scalar>& correction,
                                          bool keepdim, bool take_sqrt) {
  TORCH_CHECK(is_float_dtype(self.scalar_type()), "b200 var/std: only float32 / bfloat16 / float16 inputs have a device path");
  const auto dt = self.scalar_type();
  const std::vector<int64_t> dims = reduce_dims(self, dim);
  int64_t n = 1;
  for (int64_t d : dims) n *= self.size(d);
  Tensor x = dt == at::kFloat ? self : self.to(at::kFloat);
  Tensor mean, ss;
  if (dims.empty()) {  // 0-dim input
    mean = x.clone();
    ss = at::zeros_like(x);
  } else {
    mean = x.mean(dims, /*keepdim=*/true);
    Tensor d = x - mean;
    ss = at::mul(d, d).sum(dims, keepdim);
    if (!keepdim) mean = mean.squeeze(dims);
  }
  const double corr = correction.has_value() ? correction->toDouble() : 1.0;
  const double denom = std::max(0.0, (double)n - corr);
  Tensor v = at::div(ss, Scalar(denom));  // n - correction == 0 gives nan / inf, as on the CPU
  if (take_sqrt) v = v.sqrt();
  return {dt == at::kFloat ? v : v.to(dt), dt == at::kFloat ? mean : mean.to(dt)};
}

Tensor k_var(const Tensor& self, at::OptionalIntArrayRef dim, const std::optional<Scalar>& correction, bool keepdim) {
  return B200_DISPATCH("var", var_mean_device(self, dim, correction, keepdim, false).first,
                       B200_CPU(var_correction, self, dim, correction, keepdim));
}
Tensor k_std(const Tensor& self, at::OptionalIntArrayRef dim, const std::optional<Scalar>& correction, bool keepdim) {
  return B200_DISPATCH("std", var_mean_device(self, dim, correction, keepdim, true).first,
                       B200_CPU(std_correction, self, dim, correction, keepdim));
}
std::tuple<Tensor, Tensor> var_mean_tuple(const Tensor& self, at::OptionalIntArrayRef dim, const std::optional<Scalar>& correction,
                                          bool keepdim, bool take_sqrt) {
  auto r = var_mean_device(self, dim, correction, keepdim, take_sqrt);
  return std::make_tuple(r.first, r.second);
}
std::tuple<Tensor, Tensor> k_var_mean(const Tensor& self, at::OptionalIntArrayRef dim, const std::optional<Scalar>& correction,
                                      bool keepdim) {
  return B200_DISPATCH("var_mean", var_mean_tuple(self, dim, correction, keepdim, false),
                       B200_CPU(var_mean_correction, self, dim, correction, keepdim));
}
std::tuple<Tensor, Tensor> k_std_mean(const Tensor& self, at::OptionalIntArrayRef dim, const std::optional<Scalar>& correction,
                                      bool keepdim) {
  return B200_DISPATCH("std_mean", var_mean_tuple(self, dim, correction, keepdim, true),
                       B200_CPU(std_mean_correction, self, dim, correction, keepdim));
}

// ---- dot / addmv ---------------------------------------------------------------------------------------
Tensor dot_device(const Tensor& a, const Tensor& b) {
  TORCH_CHECK(a.dim() == 1 && b.dim() == 1 && a.size(0) == b.size(0), "dot: expected two 1-D tensors of the same length, got ",
              a.sizes(), " and ", b.sizes());
  TORCH_CHECK(a.scalar_type() == b.scalar_type() && is_float_dtype(a.scalar_type()), "b200 dot: unsupported dtypes ",
              a.scalar_type(), ", ", b.scalar_type());
  const auto dt = a.scalar_type();
  Tensor p = dt == at::kFloat ? at::mul(a, b) : at::mul(a.to(at::kFloat), b.to(at::kFloat));
  Tensor s = p.sum();
  return dt == at::kFloat ? s : s.to(dt);
}
Tensor k_dot(const Tensor& a, const Tensor& b) { return B200_DISPATCH("dot", dot_device(a, b), B200_CPU(dot, a, b)); }

// beta * self + alpha * (mat @ vec) as one GEMM with a one-column right-hand side
Tensor addmv_device(const Tensor& self, const Tensor& mat, const Tensor& vec, const Scalar& beta, const Scalar& alpha) {
  TORCH_CHECK(mat.dim() == 2 && vec.dim() == 1 && mat.size(1) == vec.size(0), "addmv: size mismatch, got ", mat.sizes(), " and ",
              vec.sizes());
  TORCH_CHECK(self.dim() <= 1, "addmv: the added tensor must be a vector or a scalar");
  const int64_t m = mat.size(0);
  Tensor bias = self.expand({m}).unsqueeze(-1);
  return at::addmm(bias, mat, vec.unsqueeze(-1), beta, alpha).squeeze(-1);
}
Tensor k_addmv(const Tensor& self, const Tensor& mat, const Tensor& vec, const Scalar& beta, const Scalar& alpha) {
  return B200_DISPATCH("addmv", addmv_device(self, mat, vec, beta, alpha), B200_CPU(addmv, self, mat, vec, beta, alpha));
}
Tensor& k_addmv_(Tensor& self, const Tensor& mat, const Tensor& vec, const Scalar& beta, const Scalar& alpha) {
  self.copy_(k_addmv(self, mat, vec, beta, alpha));
  return self;
}
Tensor& k_addmv_out(const Tensor& self, const Tensor& mat, const Tensor& vec, const Scalar& beta, const Scalar& alpha, Tensor& out) {
  Tensor r = k_addmv(self, mat, vec, beta, alpha);
  if (out.sizes() != r.sizes()) out.resize_(r.sizes());
  out.copy_(r);
  return out;
}

// ---- flip / roll: one index_select per dimension with an index built on the host -------------------------
Tensor take_along(const Tensor& x, int64_t dim, const std::vector<int64_t>& index) {
  Tensor idx = at::tensor(index, at::TensorOptions().dtype(at::kLong)).to(x.device());
  return x.index_select(dim, idx);
}
Tensor flip_device(const Tensor& self, at::IntArrayRef dims) {
  Tensor out = self;
  std::vector<bool> seen(self.dim(), false);
  for (int64_t d0 : dims) {
    const int64_t d = at::maybe_wrap_dim(d0, self.dim());
    TORCH_CHECK(!seen[d], "flip: dim ", d0, " appears more than once");
    seen[d] = true;
    const int64_t n = self.size(d);
    if (n <= 1) continue;
    std::vector<int64_t> index(n);
    for (int64_t i = 0; i < n; ++i) index[i] = n - 1 - i;
    out = take_along(out, d, index);
  }
  return out.is_same(self) ? self.clone() : out;
}
Tensor k_flip(const Tensor& self, at::IntArrayRef dims) {
  return B200_DISPATCH("flip", flip_device(self, dims), B200_CPU(flip, self, dims));
}
Tensor roll_device(const Tensor& self, at::IntArrayRef shifts, at::IntArrayRef dims) {
  TORCH_CHECK(!shifts.empty(), "roll: `shifts` required");
  if (dims.empty()) {
    TORCH_CHECK(shifts.size() == 1, "roll: shifts and dimensions must align");
    const int64_t dims0[1] = {0};
    return roll_device(self.reshape({-1}), shifts, at::IntArrayRef(dims0, 1)).view(self.sizes());
  }
  TORCH_CHECK(shifts.size() == dims.size(), "roll: shifts and dimensions must align. shifts: ", shifts.size(), ", dims: ", dims.size());
  Tensor out = self;
  for (size_t k = 0; k < dims.size(); ++k) {
    const int64_t d = at::maybe_wrap_dim(dims[k], self.dim());
    const int64_t n = self.size(d);
    if (n <= 1) continue;
    const int64_t s = ((shifts[k] % n) + n) % n;
    if (s == 0) continue;
    std::vector<int64_t> index(n);
    for (int64_t i = 0; i < n; ++i) index[i] = (i - s + n) % n;
    out = take_along(out, d, index);
  }
  return out.is_same(self) ? self.clone() : out;
}
Tensor k_roll(const Tensor& self, at::IntArrayRef shifts, at::IntArrayRef dims) {
  return B200_DISPATCH("roll", roll_device(self, shifts, dims),
                       B200_CPU_SYMINT(roll, self, c10::fromIntArrayRefSlow(shifts), dims));
}

// ---- element-wise composites -----------------------------------------------------------------------------
// compute in fp32 for 16-bit inputs, hand back the input dtype
template <typename F>
Tensor in_fp32(const Tensor& like, F&& f) {
  TORCH_CHECK(is_float_dtype(like.scalar_type()), "b200: only float32 / bfloat16 / float16 inputs have a device path here");
  Tensor r = f();
  return r.scalar_type() == like.scalar_type() ? r : r.to(like.scalar_type());
}
Tensor f32(const Tensor& t) { return t.scalar_type() == at::kFloat ? t : t.to(at::kFloat); }

Tensor elu_backward_device(const Tensor& grad, const Scalar& alpha, const Scalar& scale, const Scalar& input_scale, bool is_result,
                           const Tensor& self_or_result) {
  const double negcoef = alpha.toDouble() * scale.toDouble(), poscoef = scale.toDouble(), negiptcoef = input_scale.toDouble();
  return in_fp32(grad, [&] {
    Tensor g = f32(grad), x = f32(self_or_result);
    Tensor neg = is_result ? at::mul(g, at::add(x, Scalar(negcoef))).mul_(Scalar(negiptcoef))
                           : at::mul(g, at::exp(at::mul(x, Scalar(negiptcoef)))).mul_(Scalar(negiptcoef * negcoef));
    return at::where(at::le(x, Scalar(0.0)), neg, at::mul(g, Scalar(poscoef)));
  });
}
Tensor k_elu_backward(const Tensor& grad, const Scalar& alpha, const Scalar& scale, const Scalar& input_scale, bool is_result,
                      const Tensor& self_or_result) {
  return B200_DISPATCH("elu_backward", elu_backward_device(grad, alpha, scale, input_scale, is_result, self_or_result),
                       B200_CPU(elu_backward, grad, alpha, scale, input_scale, is_result, self_or_result));
}

Tensor hardswish_backward_device(const Tensor& grad, const Tensor& self) {
  return in_fp32(grad, [&] {
    Tensor g = f32(grad), x = f32(self);
    Tensor mid = at::mul(g, at::add(at::div(x, Scalar(3.0)), Scalar(0.5)));
    // the stock kernels' boundaries: zero up to and including -3, the slope strictly inside (-3, 3), grad from 3 on
    Tensor r = at::where(at::lt(x, Scalar(3.0)), mid, g);
    return at::where(at::le(x, Scalar(-3.0)), at::zeros_like(g), r);
  });
}
Tensor k_hardswish_backward(const Tensor& grad, const Tensor& self) {
  return B200_DISPATCH("hardswish_backward", hardswish_backward_device(grad, self), B200_CPU(hardswish_backward, grad, self));
}

Tensor logit_device(const Tensor& self, std::optional<double> eps) {
  return in_fp32(self, [&] {
    Tensor x = f32(self);
    if (eps.has_value()) x = at::clamp(x, Scalar(*eps), Scalar(1.0 - *eps));
    return at::log(at::div(x, at::rsub(x, Scalar(1.0))));
  });
}
Tensor k_logit(const Tensor& self, std::optional<double> eps) {
  return B200_DISPATCH("logit", logit_device(self, eps), B200_CPU(logit, self, eps));
}

Tensor xlogy_device(const Tensor& self, const Tensor& other) {
  const auto dt = at::result_type(self, other);
  TORCH_CHECK(is_float_dtype(dt), "b200 xlogy: only floating results have a device path");
  Tensor x = f32(self), y = f32(other);
  Tensor r = at::mul(x, at::log(y));
  r = at::where(at::eq(x, Scalar(0.0)), at::zeros_like(r), r);
  r = at::where(at::isnan(y), y.expand_as(r), r);  // a nan in `other` wins over a zero in `self`
  return dt == at::kFloat ? r : r.to(dt);
}
Tensor k_xlogy(const Tensor& self, const Tensor& other) {
  return B200_DISPATCH("xlogy", xlogy_device(self, other), B200_CPU(xlogy_Tensor, self, other));
}

// ---- group norm backward ---------------------------------------------------------------------------------
// The forward runs as a batch norm over [1, N * groups, -1] (PyTorch's composite); this is its gradient from the
// saved per-group mean and inverse standard deviation:
//   dx = rstd * (g - mean_g(g) - xhat * mean_g(g * xhat)),  g = dy * gamma,  xhat = (x - mean) * rstd
std::tuple<Tensor, Tensor, Tensor> group_norm_backward_device(const Tensor& grad_out, const Tensor& input, const Tensor& mean,
                                                              const Tensor& rstd, const std::optional<Tensor>& weight, int64_t N,
                                                              int64_t C, int64_t HxW, int64_t group, std::array<bool, 3> mask) {
  TORCH_CHECK(is_float_dtype(input.scalar_type()) && group > 0 && C % group == 0, "b200 group_norm backward: unsupported arguments");
  const auto dt = input.scalar_type();
  const int64_t D = C / group;
  const bool has_w = weight.has_value() && weight->defined();
  Tensor x = f32(input).contiguous().view({N, group, D, HxW});
  Tensor dy = f32(grad_out).contiguous().view({N, group, D, HxW});
  Tensor mu = f32(mean).contiguous().view({N, group, 1, 1}), rs = f32(rstd).contiguous().view({N, group, 1, 1});
  Tensor xhat = at::mul(at::sub(x, mu), rs);
  Tensor dx, dgamma, dbeta;
  if (mask[0]) {
    Tensor g = has_w ? at::mul(dy, f32(*weight).contiguous().view({1, group, D, 1})) : dy;
    Tensor c1 = at::mul(g, xhat).mean(std::vector<int64_t>{2, 3}, true);
    Tensor c2 = g.mean(std::vector<int64_t>{2, 3}, true);
    Tensor r = at::mul(at::sub(at::sub(g, c2), at::mul(xhat, c1)), rs).view(input.sizes());
    dx = dt == at::kFloat ? r : r.to(dt);
  }
  if (mask[1] && has_w) dgamma = at::mul(dy, xhat).sum(std::vector<int64_t>{0, 3}).view({C}).to(weight->scalar_type());
  if (mask[2] && has_w) dbeta = dy.sum(std::vector<int64_t>{0, 3}).view({C}).to(weight->scalar_type());
  return std::make_tuple(dx, dgamma, dbeta);
}
std::tuple<Tensor, Tensor, Tensor> k_group_norm_backward(const Tensor& grad_out, const Tensor& input, const Tensor& mean,
                                                         const Tensor& rstd, const std::optional<Tensor>& weight, int64_t N, int64_t C,
                                                         int64_t HxW, int64_t group, std::array<bool, 3> mask) {
  return B200_DISPATCH("native_group_norm_backward", group_norm_backward_device(grad_out, input, mean, rstd, weight, N, C, HxW, group, mask),
                       B200_CPU_SYMINT(native_group_norm_backward, grad_out, input, mean, rstd, weight, c10::SymInt(N), c10::SymInt(C),
                                       c10::SymInt(HxW), group, mask));
}

// ---- LSTM / GRU cells --------------------------------------------------------------------------------------
// torch's lstm / gru call these "fused cell" operators for every device that is not the CPU, and only CUDA ships
// kernels for them (the boxed CPU fallback cannot help: there is no CPU kernel either), so without them nn.LSTM and
// nn.GRU do not run on this device.  Here they are compositions of element-wise device kernels; the workspace that
// the forward hands to the backward is this file's own format.
//   LSTM: gates = input_gates + hidden_gates (+ biases) = [i | f | g | o]; cy = s(f) * cx + s(i) * tanh(g);
//         hy = s(o) * tanh(cy); workspace = the four activated gates.
std::tuple<Tensor, Tensor, Tensor> lstm_cell(const Tensor& input_gates, const Tensor& hidden_gates, const Tensor& cx,
                                             const std::optional<Tensor>& input_bias, const std::optional<Tensor>& hidden_bias) {
  Tensor gates = at::add(input_gates, hidden_gates);
  if (input_bias.has_value() && input_bias->defined()) gates = at::add(gates, *input_bias);
  if (hidden_bias.has_value() && hidden_bias->defined()) gates = at::add(gates, *hidden_bias);
  auto ch = gates.chunk(4, -1);
  Tensor i = at::sigmoid(ch[0]), f = at::sigmoid(ch[1]), g = at::tanh(ch[2]), o = at::sigmoid(ch[3]);
  Tensor cy = at::add(at::mul(f, cx), at::mul(i, g));
  Tensor hy = at::mul(o, at::tanh(cy));
  return std::make_tuple(hy, cy, at::cat({i, f, g, o}, -1));
}
std::tuple<Tensor, Tensor, Tensor> lstm_cell_backward(const std::optional<Tensor>& grad_hy, const std::optional<Tensor>& grad_cy,
                                                      const Tensor& cx, const Tensor& cy, const Tensor& workspace, bool has_bias) {
  auto ch = workspace.chunk(4, -1);
  const Tensor &i = ch[0], &f = ch[1], &g = ch[2], &o = ch[3];
  Tensor tc = at::tanh(cy);
  const bool has_h = grad_hy.has_value() && grad_hy->defined(), has_c = grad_cy.has_value() && grad_cy->defined();
  Tensor gh = has_h ? *grad_hy : at::zeros_like(cy);
  Tensor gc = at::mul(at::mul(gh, o), at::rsub(at::mul(tc, tc), Scalar(1.0)));  // through hy = o * tanh(cy)
  if (has_c) gc = at::add(gc, *grad_cy);
  auto dsig = [](const Tensor& s) { return at::mul(s, at::rsub(s, Scalar(1.0))); };
  Tensor di = at::mul(at::mul(gc, g), dsig(i));
  Tensor df = at::mul(at::mul(gc, cx), dsig(f));
  Tensor dg = at::mul(at::mul(gc, i), at::rsub(at::mul(g, g), Scalar(1.0)));
  Tensor d_o = at::mul(at::mul(gh, tc), dsig(o));
  Tensor grad_gates = at::cat({di, df, dg, d_o}, -1);
  Tensor grad_cx = at::mul(gc, f);
  Tensor grad_bias = has_bias ? grad_gates.sum(std::vector<int64_t>{0}) : Tensor();
  return std::make_tuple(grad_gates, grad_cx, grad_bias);
}
//   GRU: r = s(ig_r + hg_r), z = s(ig_z + hg_z), n = tanh(ig_n + r * hg_n), hy = n + z * (hx - n);
//        workspace = [r | z | n | hx | hg_n].
std::tuple<Tensor, Tensor> gru_cell(const Tensor& input_gates, const Tensor& hidden_gates, const Tensor& hx,
                                    const std::optional<Tensor>& input_bias, const std::optional<Tensor>& hidden_bias) {
  Tensor ig = (input_bias.has_value() && input_bias->defined()) ? at::add(input_gates, *input_bias) : input_gates;
  Tensor hg = (hidden_bias.has_value() && hidden_bias->defined()) ? at::add(hidden_gates, *hidden_bias) : hidden_gates;
  auto ic = ig.chunk(3, -1), hc = hg.chunk(3, -1);
  Tensor r = at::sigmoid(at::add(ic[0], hc[0])), z = at::sigmoid(at::add(ic[1], hc[1]));
  Tensor n = at::tanh(at::add(ic[2], at::mul(r, hc[2])));
  Tensor hy = at::add(n, at::mul(z, at::sub(hx, n)));
  return std::make_tuple(hy, at::cat({r, z, n, hx, hc[2]}, -1));
}
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> gru_cell_backward(const Tensor& grad_hy, const Tensor& workspace, bool has_bias) {
  auto ch = workspace.chunk(5, -1);
  const Tensor &r = ch[0], &z = ch[1], &n = ch[2], &hx = ch[3], &hn = ch[4];
  Tensor grad_hx = at::mul(grad_hy, z);
  Tensor dz = at::mul(at::mul(grad_hy, at::sub(hx, n)), at::mul(z, at::rsub(z, Scalar(1.0))));
  Tensor dn = at::mul(at::mul(grad_hy, at::rsub(z, Scalar(1.0))), at::rsub(at::mul(n, n), Scalar(1.0)));
  Tensor dr = at::mul(at::mul(dn, hn), at::mul(r, at::rsub(r, Scalar(1.0))));
  Tensor grad_input_gates = at::cat({dr, dz, dn}, -1);
  Tensor grad_hidden_gates = at::cat({dr, dz, at::mul(dn, r)}, -1);
  Tensor gib, ghb;
  if (has_bias) {
    gib = grad_input_gates.sum(std::vector<int64_t>{0});
    ghb = grad_hidden_gates.sum(std::vector<int64_t>{0});
  }
  return std::make_tuple(grad_input_gates, grad_hidden_gates, grad_hx, gib, ghb);
}

}  // namespace

// registered under host simulation as well: the boxed CPU fallback has no kernel to fall back to
TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_thnn_fused_lstm_cell", TORCH_FN(lstm_cell));
  m.impl("_thnn_fused_lstm_cell_backward_impl", TORCH_FN(lstm_cell_backward));
  m.impl("_thnn_fused_gru_cell", TORCH_FN(gru_cell));
  m.impl("_thnn_fused_gru_cell_backward", TORCH_FN(gru_cell_backward));
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("var.correction", TORCH_FN(k_var));
  m.impl("std.correction", TORCH_FN(k_std));
  m.impl("var_mean.correction", TORCH_FN(k_var_mean));
  m.impl("std_mean.correction", TORCH_FN(k_std_mean));
  m.impl("dot", TORCH_FN(k_dot));
  m.impl("addmv", TORCH_FN(k_addmv));
  m.impl("addmv_", TORCH_FN(k_addmv_));
  m.impl("addmv.out", TORCH_FN(k_addmv_out));
  m.impl("flip", TORCH_FN(k_flip));
  m.impl("roll", TORCH_FN(k_roll));
  m.impl("elu_backward", TORCH_FN(k_elu_backward));
  m.impl("hardswish_backward", TORCH_FN(k_hardswish_backward));
  m.impl("logit", TORCH_FN(k_logit));
  m.impl("xlogy.Tensor", TORCH_FN(k_xlogy));
  m.impl("native_group_norm_backward", TORCH_FN(k_group_norm_backward));
}

}  // namespace ops
}  // namespace catch_b200
