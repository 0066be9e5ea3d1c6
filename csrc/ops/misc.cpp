// Embedding, index_select, random number operators, dropout, the device dump
// op and the fused optimizer steps.
//
// Parity: index_select.cpp / the generator of the reference; embedding, dropout
// and the fused optimizers are new (the reference runs them through the CPU
// fallback or as many small element-wise launches).
#include <ATen/core/op_registration/op_registration.h>
#include <ATen/CPUGeneratorImpl.h>
#include "../runtime/generator.h"
#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

bool f_ok(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf; }

Tensor embedding_device(const Tensor& weight, const Tensor& indices_in, int64_t padding_idx) {
  TORCH_CHECK(weight.dim() == 2 && (indices_in.scalar_type() == at::kLong || indices_in.scalar_type() == at::kInt),
              "b200 embedding: weight must be 2-D and indices int64 or int32");
  const Tensor indices = indices_in.scalar_type() == at::kInt ? indices_in.to(at::kLong) : indices_in;  // the kernel reads int64
  OpScope scope("embedding", weight);
  Tensor w = weight.contiguous(), idx = indices.contiguous();
  std::vector<int64_t> shape(indices.sizes().begin(), indices.sizes().end());
  shape.push_back(w.size(1));
  Tensor out = empty_b200(shape, w.scalar_type(), w.device().index());
  B200_KERNEL_CHECK(b200_index_select_rows(w.data_ptr(), (int)w.element_size(), i64ptr(idx), idx.numel(), w.size(1),
                                           w.size(0), out.data_ptr(), scope.stream()));
  (void)padding_idx;
  return out;
}
Tensor k_embedding(const Tensor& weight, const Tensor& indices, c10::SymInt padding_idx, bool scale, bool sparse) {
  check_same_device("embedding", weight, indices);
  return B200_DISPATCH("embedding", embedding_device(weight, indices, padding_idx.expect_int()),
                       B200_CPU_SYMINT(embedding, weight, indices, padding_idx, scale, sparse));
}
Tensor embedding_bwd_device(const Tensor& grad, const Tensor& indices_in, int64_t num_weights, int64_t padding_idx, bool scale) {
  const Tensor indices = indices_in.scalar_type() == at::kInt ? indices_in.to(at::kLong) : indices_in;
  TORCH_CHECK(!scale && f_ok(grad.scalar_type()) && indices.scalar_type() == at::kLong, "b200 embedding_backward: unsupported arguments");
  OpScope scope("embedding_dense_backward", grad);
  Tensor g = grad.contiguous().view({-1, grad.size(-1)}), idx = indices.contiguous();
  // accumulate in fp32 for accuracy, then cast
  Tensor acc = at::zeros({num_weights, g.size(1)}, grad.options().dtype(at::kFloat));
  B200_KERNEL_CHECK(b200_embedding_bwd(g.data_ptr(), to_b200_dtype(g.scalar_type()), i64ptr(idx), idx.numel(), (int)g.size(1),
                                       padding_idx, acc.data_ptr(), B200_F32, scope.stream()));
  return grad.scalar_type() == at::kFloat ? acc : acc.to(grad.scalar_type());
}
Tensor k_embedding_dense_backward(const Tensor& grad, const Tensor& indices, c10::SymInt num_weights, c10::SymInt padding_idx,
                                  bool scale) {
  return B200_DISPATCH("embedding_dense_backward",
                       embedding_bwd_device(grad, indices, num_weights.expect_int(), padding_idx.expect_int(), scale),
                       B200_CPU_SYMINT(embedding_dense_backward, grad, indices, num_weights, padding_idx, scale));
}

Tensor index_select_device(const Tensor& self, int64_t dim, const Tensor& index_in) {
  TORCH_CHECK(index_in.dim() <= 1 && (index_in.scalar_type() == at::kLong || index_in.scalar_type() == at::kInt),
              "b200 index_select: index must be a 1-D int64 or int32 tensor");
  const Tensor index = index_in.scalar_type() == at::kInt ? index_in.to(at::kLong) : index_in;  // the kernel reads int64
  dim = at::maybe_wrap_dim(dim, self.dim());
  OpScope scope("index_select", self);
  if (self.dim() == 0) return self.clone();
  Tensor x = self.movedim(dim, 0).contiguous();
  Tensor idx = index.contiguous().view({-1});
  std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
  const int64_t n_src = shape[0];
  shape[0] = idx.numel();
  Tensor out = empty_b200(shape, self.scalar_type(), self.device().index());
  const int64_t row = n_src ? x.numel() / n_src : 0;
  B200_KERNEL_CHECK(b200_index_select_rows(x.data_ptr(), (int)x.element_size(), i64ptr(idx), idx.numel(), row, n_src,
                                           out.data_ptr(), scope.stream()));
  return out.movedim(0, dim).contiguous();  // a contiguous result, as from the stock kernel
}
Tensor k_index_select(const Tensor& self, int64_t dim, const Tensor& index) {
  check_same_device("index_select", self, index);
  return B200_DISPATCH("index_select", index_select_device(self, dim, index), B200_CPU(index_select, self, dim, index));
}

// ---- random ---------------------------------------------------------------------------
std::pair<uint64_t, uint64_t> philox(std::optional<at::Generator> gen, const Tensor& t, uint64_t n) {
  auto g = at::get_generator_or_default<B200GeneratorImpl>(gen, getDefaultB200Generator(t.device().index()));
  std::lock_guard<std::mutex> lock(g->mutex_);
  return g->philox_engine_inputs(n);
}
Tensor& rng_fill(Tensor& self, std::optional<at::Generator> gen, int mode, double a, double b) {
  if (self.numel() == 0) return self;
  TORCH_CHECK(f_ok(self.scalar_type()) || self.scalar_type() == at::kDouble || (mode == 2),
              "b200 random fill: unsupported dtype ", self.scalar_type());
  OpScope scope("random_fill", self);
  Tensor dst = self.is_contiguous() ? self : at::empty_like(self, at::MemoryFormat::Contiguous);
  auto so = philox(gen, self, (uint64_t)dst.numel());
  const int dt = to_b200_dtype(dst.scalar_type());
  if (mode == 0) B200_KERNEL_CHECK(b200_rng_uniform(dst.data_ptr(), dt, dst.numel(), so.first, so.second, a, b, scope.stream()));
  else if (mode == 1) B200_KERNEL_CHECK(b200_rng_normal(dst.data_ptr(), dt, dst.numel(), so.first, so.second, a, b, scope.stream()));
  else B200_KERNEL_CHECK(b200_rng_bernoulli(dst.data_ptr(), dt, dst.numel(), so.first, so.second, a, scope.stream()));
  if (!dst.is_same(self)) self.copy_(dst);
  return self;
}
Tensor& k_uniform_(Tensor& self, double from, double to, std::optional<at::Generator> gen) {
  return rng_fill(self, gen, 0, from, to);
}
Tensor& k_normal_(Tensor& self, double mean, double std, std::optional<at::Generator> gen) {
  return rng_fill(self, gen, 1, mean, std);
}
Tensor& k_bernoulli_float_(Tensor& self, double p, std::optional<at::Generator> gen) {
  return rng_fill(self, gen, 2, p, 0);
}
// CPU path (host simulation / forced CPU dispatch): the values come from a CPU
// generator seeded from this device's (seed, offset) pair, so torch.blackwell
// seeding and RNG-state save / restore behave the same with and without a GPU.
Tensor& rng_fill_cpu(Tensor& self, std::optional<at::Generator> gen, int mode, double a, double b) {
  if (self.numel() == 0) return self;
  auto so = philox(gen, self, (uint64_t)self.numel());
  at::Generator cpu_gen = at::detail::createCPUGenerator(so.first * 0x9E3779B97F4A7C15ull + so.second);
  Tensor host = at::empty(self.sizes(), self.options().device(at::kCPU));
  if (mode == 0) host.uniform_(a, b, cpu_gen);
  else if (mode == 1) host.normal_(a, b, cpu_gen);
  else host.bernoulli_(a, cpu_gen);
  self.copy_(host);
  return self;
}
Tensor& c_uniform_(Tensor& self, double from, double to, std::optional<at::Generator> gen) { return rng_fill_cpu(self, gen, 0, from, to); }
Tensor& c_normal_(Tensor& self, double mean, double std, std::optional<at::Generator> gen) { return rng_fill_cpu(self, gen, 1, mean, std); }
Tensor& c_bernoulli_float_(Tensor& self, double p, std::optional<at::Generator> gen) { return rng_fill_cpu(self, gen, 2, p, 0); }
std::tuple<Tensor, Tensor> c_native_dropout(const Tensor& input, double p, std::optional<bool> train) {
  if (!train.value_or(true) || p == 0.0 || input.numel() == 0)
    return {input.clone(), at::ones_like(input, input.options().dtype(at::kBool))};
  Tensor keep = at::empty(input.sizes(), input.options().dtype(at::kFloat));
  rng_fill_cpu(keep, std::nullopt, 2, 1.0 - p, 0);
  Tensor mask = keep.to(at::kBool);
  return {input * mask.to(input.scalar_type()) * (p < 1.0 ? 1.0 / (1.0 - p) : 0.0), mask};
}

std::tuple<Tensor, Tensor> k_native_dropout(const Tensor& input, double p, std::optional<bool> train) {
  if (!train.value_or(true) || p == 0.0 || input.numel() == 0) {
    return {input.clone(), at::ones_like(input, input.options().dtype(at::kBool))};
  }
  TORCH_CHECK(f_ok(input.scalar_type()), "b200 dropout: unsupported dtype ", input.scalar_type());
  OpScope scope("native_dropout", input);
  Tensor x = input.contiguous();
  Tensor y = at::empty_like(x), mask = at::empty_like(x, x.options().dtype(at::kBool));
  auto so = philox(std::nullopt, input, (uint64_t)x.numel());
  B200_KERNEL_CHECK(b200_dropout_fwd(x.data_ptr(), to_b200_dtype(x.scalar_type()), x.numel(), so.first, so.second, (float)p,
                                     y.data_ptr(), static_cast<unsigned char*>(mask.data_ptr()), scope.stream()));
  return {y, mask};
}
Tensor k_native_dropout_backward(const Tensor& grad, const Tensor& mask, double scale) {
  if (f_ok(grad.scalar_type()) && mask.scalar_type() == at::kBool && grad.is_contiguous() && mask.is_contiguous() &&
      grad.numel() == mask.numel() && is_b200(grad) && !use_cpu_path()) {
    OpScope scope("native_dropout_backward", grad);
    Tensor dx = at::empty_like(grad);
    B200_KERNEL_CHECK(b200_dropout_bwd(grad.data_ptr(), static_cast<const unsigned char*>(mask.data_ptr()),
                                       to_b200_dtype(grad.scalar_type()), grad.numel(), (float)scale, dx.data_ptr(), scope.stream()));
    return dx;
  }
  return grad * mask.to(grad.scalar_type()) * scale;
}

}  // namespace

// ---- fused transformer residual block ---------------------------------------------------------
// s = residual + dropout(h); y = layer_norm(s).  Returns (y, s, mask, mean, rstd); mask has one byte per four elements.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> dropout_add_layer_norm(
    const at::Tensor& h, const at::Tensor& residual, const std::optional<at::Tensor>& weight, const std::optional<at::Tensor>& bias,
    double p, bool training, double eps) {
  TORCH_CHECK(h.sizes() == residual.sizes() && h.scalar_type() == residual.scalar_type() && f_ok(h.scalar_type()) && h.dim() >= 1,
              "dropout_add_layer_norm: h and residual must match");
  const int64_t cols = h.size(-1), rows = cols ? h.numel() / cols : 0;
  if (use_cpu_path()) {
    // Host path (host simulation, force-CPU mode): the same five results from ordinary tensor operations; the mask
    // holds one byte per element here (the device packs it), which only the matching backward below reads.
    const bool drop = training && p > 0.0;
    at::Tensor hf = h.to(at::kFloat).reshape({rows, cols});
    at::Tensor mask = at::empty({0}, h.options().dtype(at::kByte));
    if (drop) {
      at::Tensor keep = at::bernoulli(at::full({rows, cols}, 1.0 - p, hf.options()));
      hf = hf * keep / (1.0 - p);
      mask = keep.to(at::kByte).reshape({-1});
    }
    at::Tensor sf = residual.to(at::kFloat).reshape({rows, cols}) + hf;
    at::Tensor mean = sf.mean(std::vector<int64_t>{1});
    at::Tensor var = (sf - mean.unsqueeze(1)).square().mean(std::vector<int64_t>{1});
    at::Tensor rstd = (var + eps).rsqrt();
    at::Tensor yf = (sf - mean.unsqueeze(1)) * rstd.unsqueeze(1);
    if (weight.has_value() && weight->defined()) yf = yf * weight->to(at::kFloat);
    if (bias.has_value() && bias->defined()) yf = yf + bias->to(at::kFloat);
    return {yf.to(h.scalar_type()).reshape(h.sizes()), sf.to(h.scalar_type()).reshape(h.sizes()), mask, mean, rstd};
  }
  TORCH_CHECK(is_b200(h), "dropout_add_layer_norm: operands must be on the device");
  TORCH_CHECK(cols % 4 == 0 && cols <= b200_dropout_add_layernorm_max_cols(), "dropout_add_layer_norm: unsupported row length ", cols);
  OpScope scope("dropout_add_layer_norm", h);
  at::Tensor hc = h.contiguous(), rc = residual.contiguous();
  at::Tensor y = at::empty_like(hc), s = at::empty_like(hc);
  auto fopt = h.options().dtype(at::kFloat);
  at::Tensor mean = at::empty({rows}, fopt), rstd = at::empty({rows}, fopt);
  const float pp = training ? (float)p : 0.f;
  at::Tensor mask = at::empty({pp > 0.f ? rows * cols / 4 : 0}, h.options().dtype(at::kByte));
  std::pair<uint64_t, uint64_t> so{0, 0};
  if (pp > 0.f) so = philox(std::nullopt, h, (uint64_t)hc.numel());
  at::Tensor wk, bk;
  const void* gamma = nullptr;
  const void* beta = nullptr;
  int pdt = B200_F32;
  if (weight.has_value() && weight->defined()) { wk = weight->contiguous(); gamma = wk.data_ptr(); pdt = to_b200_dtype(wk.scalar_type()); }
  if (bias.has_value() && bias->defined()) {
    bk = bias->contiguous();
    TORCH_CHECK(!gamma || bk.scalar_type() == wk.scalar_type(), "dropout_add_layer_norm: weight and bias dtypes differ");
    beta = bk.data_ptr(); pdt = to_b200_dtype(bk.scalar_type());
  }
  B200_KERNEL_CHECK(b200_dropout_add_layernorm_fwd(hc.data_ptr(), rc.data_ptr(), to_b200_dtype(h.scalar_type()), rows, (int)cols, pp,
                                                   so.first, so.second, gamma, beta, pdt, (float)eps, y.data_ptr(), s.data_ptr(),
                                                   mask.numel() ? static_cast<unsigned char*>(mask.data_ptr()) : nullptr,
                                                   mean.data_ptr<float>(), rstd.data_ptr<float>(), scope.stream()));
  return {y, s, mask, mean, rstd};
}

// (ds, dh, dgamma, dbeta); ds is also the gradient of the residual input
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> dropout_add_layer_norm_backward(
    const at::Tensor& dy, const at::Tensor& s, const at::Tensor& mask, const std::optional<at::Tensor>& weight,
    const at::Tensor& mean, const at::Tensor& rstd, double p) {
  const int64_t cols = s.size(-1), rows = cols ? s.numel() / cols : 0;
  if (use_cpu_path()) {  // host path: see the forward; `mask` has one byte per element here
    at::Tensor g = dy.to(at::kFloat).reshape({rows, cols});
    at::Tensor xhat = (s.to(at::kFloat).reshape({rows, cols}) - mean.unsqueeze(1)) * rstd.unsqueeze(1);
    at::Tensor gy = (weight.has_value() && weight->defined()) ? g * weight->to(at::kFloat) : g;
    at::Tensor dgamma = (g * xhat).sum(std::vector<int64_t>{0}), dbeta = g.sum(std::vector<int64_t>{0});
    at::Tensor c1 = (gy * xhat).mean(std::vector<int64_t>{1}, true), c2 = gy.mean(std::vector<int64_t>{1}, true);
    at::Tensor ds = (gy - c2 - xhat * c1) * rstd.unsqueeze(1);
    at::Tensor dh = ds;
    if (mask.numel() > 0) {
      TORCH_CHECK(mask.numel() == rows * cols, "dropout_add_layer_norm_backward (host path): expects the host path's mask");
      dh = ds * mask.to(at::kFloat).reshape({rows, cols}) / (1.0 - p);
    }
    return {ds.to(s.scalar_type()).reshape(s.sizes()), dh.to(s.scalar_type()).reshape(s.sizes()), dgamma, dbeta};
  }
  TORCH_CHECK(is_b200(dy), "dropout_add_layer_norm_backward: operands must be on the device");
  OpScope scope("dropout_add_layer_norm_backward", dy);
  at::Tensor g = dy.contiguous();
  TORCH_CHECK(g.scalar_type() == s.scalar_type() && g.numel() == s.numel() && s.is_contiguous(), "dropout_add_layer_norm_backward: shape / dtype mismatch");
  at::Tensor ds = at::empty_like(s), dh = at::empty_like(s);
  auto fopt = s.options().dtype(at::kFloat);
  at::Tensor dgamma = at::zeros({cols}, fopt), dbeta = at::zeros({cols}, fopt);
  at::Tensor wk;
  const void* gamma = nullptr;
  int pdt = B200_F32;
  if (weight.has_value() && weight->defined()) { wk = weight->contiguous(); gamma = wk.data_ptr(); pdt = to_b200_dtype(wk.scalar_type()); }
  const bool has_mask = mask.numel() > 0;
  B200_KERNEL_CHECK(b200_dropout_add_layernorm_bwd(g.data_ptr(), s.data_ptr(), has_mask ? static_cast<const unsigned char*>(mask.data_ptr()) : nullptr,
                                                   to_b200_dtype(s.scalar_type()), rows, (int)cols, has_mask ? (float)p : 0.f, gamma, pdt,
                                                   mean.data_ptr<float>(), rstd.data_ptr<float>(), ds.data_ptr(), dh.data_ptr(),
                                                   dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), scope.stream()));
  return {ds, dh, dgamma, dbeta};
}

// ---- custom ops (namespace catch_b200) ------------------------------------------------------
bool dump_tensor_device(const at::Tensor& t) {
  if (!is_b200(t) || use_cpu_path()) {
    std::cout << t << std::endl;
    return true;
  }
  OpScope scope("dump", t);
  at::Tensor x = t.contiguous();
  if (x.scalar_type() != at::kFloat && x.scalar_type() != at::kHalf && x.scalar_type() != at::kBFloat16) x = x.to(at::kFloat);
  B200_KERNEL_CHECK(b200_dump_device(x.data_ptr(), to_b200_dtype(x.scalar_type()), x.numel(), scope.stream()));
  scope.queue().synchronize();
  return true;
}

static void fill_opt_tensors(B200OptTensors& T, at::TensorList params, at::TensorList grads, at::TensorList s1,
                             at::TensorList s2, at::TensorList lowp, size_t begin, size_t end) {
  std::memset(&T, 0, sizeof(T));
  T.count = (int)(end - begin);
  for (size_t i = begin; i < end; ++i) {
    const size_t k = i - begin;
    // the update is element-wise, so any dense layout works as long as parameter,
    // gradient and state share it
    TORCH_CHECK(params[i].scalar_type() == at::kFloat && params[i].is_non_overlapping_and_dense(),
                "fused optimizer: parameters must be dense fp32 tensors");
    TORCH_CHECK(grads[i].strides() == params[i].strides() && grads[i].sizes() == params[i].sizes(),
                "fused optimizer: gradient layout differs from the parameter's");
    TORCH_CHECK(s1.empty() || s1[i].strides() == params[i].strides(), "fused optimizer: state layout differs from the parameter's");
    TORCH_CHECK(s2.empty() || s2[i].strides() == params[i].strides(), "fused optimizer: state layout differs from the parameter's");
    T.param[k] = params[i].data_ptr();
    T.grad[k] = grads[i].data_ptr();
    T.state1[k] = s1.empty() ? nullptr : s1[i].data_ptr();
    T.state2[k] = s2.empty() ? nullptr : s2[i].data_ptr();
    T.lowp[k] = lowp.empty() ? nullptr : lowp[i].data_ptr();
    T.numel[k] = params[i].numel();
  }
  T.grad_dtype = to_b200_dtype(grads[begin].scalar_type());
  T.lowp_dtype = lowp.empty() ? B200_BF16 : to_b200_dtype(lowp[begin].scalar_type());
}

void fused_sgd_step(at::TensorList params, at::TensorList grads, at::TensorList momentum_bufs, at::TensorList lowp,
                    double lr, double momentum, double dampening, double weight_decay, bool nesterov, bool first_step,
                    double grad_scale) {
  if (params.empty()) return;
  TORCH_CHECK(params.size() == grads.size(), "fused_sgd_step: list length mismatch");
  if (use_cpu_path()) {
    for (size_t i = 0; i < params.size(); ++i) {
      at::Tensor p = params[i];
      at::Tensor d = grads[i].to(at::kFloat) * grad_scale + p * weight_decay;
      if (momentum != 0.0) {
        at::Tensor buf = momentum_bufs[i];
        if (first_step) buf.copy_(d); else buf.mul_(momentum).add_(d, 1.0 - dampening);
        d = nesterov ? d + buf * momentum : buf;
      }
      p.sub_(d * lr);
      if (!lowp.empty()) lowp[i].copy_(p);
    }
    return;
  }
  OpScope scope("fused_sgd_step", params[0]);
  for (size_t b = 0; b < params.size(); b += B200_OPT_MAX_TENSORS) {
    const size_t e = std::min(params.size(), b + (size_t)B200_OPT_MAX_TENSORS);
    B200OptTensors T;
    fill_opt_tensors(T, params, grads, momentum != 0.0 ? momentum_bufs : at::TensorList(), {}, lowp, b, e);
    B200_KERNEL_CHECK(b200_sgd_step(&T, (float)lr, (float)momentum, (float)dampening, (float)weight_decay, nesterov,
                                    first_step, (float)grad_scale, scope.stream()));
  }
}

void fused_adamw_step(at::TensorList params, at::TensorList grads, at::TensorList exp_avg, at::TensorList exp_avg_sq,
                      at::TensorList lowp, double lr, double beta1, double beta2, double eps, double weight_decay,
                      int64_t step, double grad_scale, bool adam_l2_mode) {
  if (params.empty()) return;
  if (use_cpu_path()) {
    const double bc1 = 1.0 - std::pow(beta1, (double)step), bc2 = std::sqrt(1.0 - std::pow(beta2, (double)step));
    for (size_t i = 0; i < params.size(); ++i) {
      at::Tensor p = params[i];
      at::Tensor g = grads[i].to(at::kFloat) * grad_scale;
      if (adam_l2_mode) g = g + p * weight_decay; else p.mul_(1.0 - lr * weight_decay);
      exp_avg[i].mul_(beta1).add_(g, 1.0 - beta1);
      exp_avg_sq[i].mul_(beta2).addcmul_(g, g, 1.0 - beta2);
      at::Tensor denom = exp_avg_sq[i].sqrt() / bc2 + eps;
      p.addcdiv_(exp_avg[i], denom, -lr / bc1);
      if (!lowp.empty()) lowp[i].copy_(p);
    }
    return;
  }
  OpScope scope("fused_adamw_step", params[0]);
  for (size_t b = 0; b < params.size(); b += B200_OPT_MAX_TENSORS) {
    const size_t e = std::min(params.size(), b + (size_t)B200_OPT_MAX_TENSORS);
    B200OptTensors T;
    fill_opt_tensors(T, params, grads, exp_avg, exp_avg_sq, lowp, b, e);
    B200_KERNEL_CHECK(b200_adamw_step(&T, (float)lr, (float)beta1, (float)beta2, (float)eps, (float)weight_decay, step,
                                      (float)grad_scale, adam_l2_mode, scope.stream()));
  }
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) {
    m.impl("uniform_", TORCH_FN(c_uniform_));
    m.impl("normal_", TORCH_FN(c_normal_));
    m.impl("bernoulli_.float", TORCH_FN(c_bernoulli_float_));
    m.impl("native_dropout", TORCH_FN(c_native_dropout));
    return;
  }
  m.impl("embedding", TORCH_FN(k_embedding));
  m.impl("embedding_dense_backward", TORCH_FN(k_embedding_dense_backward));
  m.impl("index_select", TORCH_FN(k_index_select));
  m.impl("uniform_", TORCH_FN(k_uniform_));
  m.impl("normal_", TORCH_FN(k_normal_));
  m.impl("bernoulli_.float", TORCH_FN(k_bernoulli_float_));
  m.impl("native_dropout", TORCH_FN(k_native_dropout));
  m.impl("native_dropout_backward", TORCH_FN(k_native_dropout_backward));
}

}  // namespace ops
}  // namespace catch_b200
