// Batch normalisation and layer normalisation operators.
//
// Parity: torch_mlu/csrc/aten/operators/cnnl/native_batch_norm.cpp:77,
// native_batch_norm_backward.cpp:85 (train / eval, 2-5-D inputs viewed as
// channels-last 4-D).  LayerNorm is new (the reference has no device kernel).
#include <map>
#include <mutex>

#include "../runtime/caching_allocator.h"
#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

struct RowsView {
  Tensor t;       // dense tensor whose memory is [rows, C]
  int64_t rows, C;
  bool channels_last_4d;
};

// Memory view [rows, C] of an [N, C, *] tensor (copying to channels-last if needed).
RowsView rows_view(const Tensor& x) {
  RowsView v;
  v.C = x.size(1);
  v.rows = v.C ? x.numel() / v.C : 0;
  v.channels_last_4d = false;
  if (x.dim() == 2) {
    v.t = x.contiguous();
  } else if (x.dim() == 4) {
    v.t = x.contiguous(at::MemoryFormat::ChannelsLast);
    v.channels_last_4d = true;
  } else if (x.dim() == 5) {
    v.t = x.contiguous(at::MemoryFormat::ChannelsLast3d);
  } else {
    // [N, C, L] -> treat as [N, C, L, 1]
    v.t = x.unsqueeze(-1).contiguous(at::MemoryFormat::ChannelsLast).squeeze(-1);
  }
  return v;
}

Tensor like_rows(const RowsView& v, const Tensor& x, at::ScalarType dt) {
  // allocate an output with the same memory layout as v.t
  return at::empty_strided(v.t.sizes(), v.t.strides(), x.options().dtype(dt));
}

// Results follow the memory format of the input, as the stock kernels' do: channels-last inputs keep the layout
// the kernels work in, anything else gets a contiguous result (composites such as group_norm call view() on it).
Tensor in_format_of(const Tensor& t, const Tensor& like) {
  if (!t.defined() || t.numel() == 0) return t;
  if (like.dim() == 4 && like.suggest_memory_format() == at::MemoryFormat::ChannelsLast) return t;
  if (like.dim() == 5 && like.suggest_memory_format() == at::MemoryFormat::ChannelsLast3d) return t;
  return t.contiguous();
}

bool bn_dtype_ok(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf; }

const void* opt_ptr(const std::optional<Tensor>& t, Tensor& keep) {
  if (t.has_value() && t->defined()) {
    keep = t->contiguous();
    return keep.data_ptr();
  }
  return nullptr;
}

std::tuple<Tensor, Tensor, Tensor> batch_norm_device(const Tensor& input, const std::optional<Tensor>& weight,
                                                     const std::optional<Tensor>& bias,
                                                     const std::optional<Tensor>& running_mean,
                                                     const std::optional<Tensor>& running_var, bool training,
                                                     double momentum, double eps) {
  TORCH_CHECK(input.dim() >= 2 && bn_dtype_ok(input.scalar_type()), "b200 batch_norm: unsupported input ", describe(input));
  OpScope scope("native_batch_norm", input);
  RowsView v = rows_view(input);
  const int C = (int)v.C;
  const int vec = input.scalar_type() == at::kFloat ? 4 : 8;
  TORCH_CHECK(C % vec == 0, "b200 batch_norm: channels must be a multiple of ", vec);
  Tensor out = like_rows(v, input, input.scalar_type());
  auto fopt = input.options().dtype(at::kFloat);
  Tensor wk, bk, rmk, rvk;
  const void* gamma = opt_ptr(weight, wk);
  const void* beta = opt_ptr(bias, bk);
  int pdt = B200_F32;
  if (gamma) pdt = to_b200_dtype(wk.scalar_type());
  else if (beta) pdt = to_b200_dtype(bk.scalar_type());
  if (gamma && beta) TORCH_CHECK(wk.scalar_type() == bk.scalar_type(), "batch_norm: weight and bias dtypes differ");
  const int xdt = to_b200_dtype(input.scalar_type());
  Tensor save_mean, save_invstd;
  if (training) {
    save_mean = at::empty({C}, fopt);
    save_invstd = at::empty({C}, fopt);
    if (input.numel() == 0) return {out, save_mean, save_invstd};
    Tensor sums = at::zeros({2 * C}, input.options().dtype(at::kDouble));
    B200_KERNEL_CHECK(b200_bn_stats(v.t.data_ptr(), xdt, v.rows, C, sums.data_ptr<double>(), scope.stream()));
    void* rm = nullptr;
    void* rv = nullptr;
    int rdt = B200_F32;
    if (running_mean.has_value() && running_mean->defined()) {
      TORCH_CHECK(running_mean->is_contiguous() && running_var->is_contiguous(), "batch_norm: running stats must be contiguous");
      rm = running_mean->data_ptr();
      rv = running_var->data_ptr();
      rdt = to_b200_dtype(running_mean->scalar_type());
    }
    B200_KERNEL_CHECK(b200_bn_finalize(sums.data_ptr<double>(), v.rows, C, (float)eps, (float)momentum,
                                       save_mean.data_ptr<float>(), save_invstd.data_ptr<float>(), rm, rv, rdt,
                                       scope.stream()));
    B200_KERNEL_CHECK(b200_bn_apply(v.t.data_ptr(), xdt, out.data_ptr(), xdt, v.rows, C, save_mean.data_ptr(), B200_F32,
                                    save_invstd.data_ptr<float>(), gamma, beta, pdt, nullptr, 0, 0, scope.stream()));
  } else {
    TORCH_CHECK(running_mean.has_value() && running_mean->defined() && running_var.has_value() && running_var->defined(),
                "batch_norm: running statistics are required in evaluation mode");
    save_mean = at::empty({0}, fopt);
    save_invstd = at::empty({0}, fopt);
    if (input.numel() == 0) return {out, save_mean, save_invstd};
    Tensor invstd = at::empty({C}, fopt);
    Tensor rm = running_mean->contiguous(), rv = running_var->contiguous();
    B200_KERNEL_CHECK(b200_bn_invstd_from_var(rv.data_ptr(), to_b200_dtype(rv.scalar_type()), C, (float)eps,
                                              invstd.data_ptr<float>(), scope.stream()));
    B200_KERNEL_CHECK(b200_bn_apply(v.t.data_ptr(), xdt, out.data_ptr(), xdt, v.rows, C, rm.data_ptr(),
                                    to_b200_dtype(rm.scalar_type()), invstd.data_ptr<float>(), gamma, beta, pdt, nullptr,
                                    0, 0, scope.stream()));
  }
  return {in_format_of(out, input), save_mean, save_invstd};
}

// The host path of batch norm.  The boxed CPU fallback cannot be used for it: the schema of native_batch_norm does not
// mark the running statistics as written, so the fallback would update copies and drop them (a module would train
// with frozen statistics under host simulation, and on the device whenever a channel count sends it here).
std::tuple<Tensor, Tensor, Tensor> batch_norm_on_cpu(const Tensor& input, const std::optional<Tensor>& weight,
                                                   const std::optional<Tensor>& bias,
                                                   const std::optional<Tensor>& running_mean,
                                                   const std::optional<Tensor>& running_var, bool training, double momentum,
                                                   double eps) {
  auto host = [](const std::optional<Tensor>& t) {
    return (t.has_value() && t->defined()) ? std::optional<Tensor>(t->cpu()) : std::optional<Tensor>();
  };
  std::optional<Tensor> rm = host(running_mean), rv = host(running_var);
  auto r = at::native_batch_norm(input.cpu(), host(weight), host(bias), rm, rv, training, momentum, eps);
  if (training && rm.has_value() && rv.has_value()) {
    running_mean->copy_(*rm);
    running_var->copy_(*rv);
  }
  const auto dev = input.device();
  return {std::get<0>(r).to(dev), std::get<1>(r).to(dev), std::get<2>(r).to(dev)};
}

std::tuple<Tensor, Tensor, Tensor> k_native_batch_norm(const Tensor& input, const std::optional<Tensor>& weight,
                                                     const std::optional<Tensor>& bias,
                                                     const std::optional<Tensor>& running_mean,
                                                     const std::optional<Tensor>& running_var, bool training,
                                                     double momentum, double eps) {
  check_same_device("batch_norm", input, weight, bias, running_mean, running_var);
  return B200_DISPATCH("native_batch_norm",
                       batch_norm_device(input, weight, bias, running_mean, running_var, training, momentum, eps),
                       batch_norm_on_cpu(input, weight, bias, running_mean, running_var, training, momentum, eps));
}

std::tuple<Tensor, Tensor, Tensor> bn_legit(const Tensor& input, const std::optional<Tensor>& weight,
                                            const std::optional<Tensor>& bias, Tensor& running_mean, Tensor& running_var,
                                            bool training, double momentum, double eps) {
  return k_native_batch_norm(input, weight, bias, running_mean, running_var, training, momentum, eps);
}
std::tuple<Tensor, Tensor, Tensor> bn_legit_no_stats(const Tensor& input, const std::optional<Tensor>& weight,
                                                     const std::optional<Tensor>& bias, bool training, double momentum,
                                                     double eps) {
  return k_native_batch_norm(input, weight, bias, std::nullopt, std::nullopt, training, momentum, eps);
}
std::tuple<Tensor, Tensor, Tensor> bn_legit_no_training(const Tensor& input, const std::optional<Tensor>& weight,
                                                        const std::optional<Tensor>& bias, const Tensor& running_mean,
                                                        const Tensor& running_var, double momentum, double eps) {
  return k_native_batch_norm(input, weight, bias, running_mean, running_var, false, momentum, eps);
}

std::tuple<Tensor, Tensor, Tensor> batch_norm_backward_device(
    const Tensor& grad_out, const Tensor& input, const std::optional<Tensor>& weight,
    const std::optional<Tensor>& running_mean, const std::optional<Tensor>& running_var,
    const std::optional<Tensor>& save_mean, const std::optional<Tensor>& save_invstd, bool train, double eps,
    std::array<bool, 3> mask) {
  TORCH_CHECK(bn_dtype_ok(input.scalar_type()) && grad_out.scalar_type() == input.scalar_type(),
              "b200 batch_norm_backward: unsupported dtypes");
  OpScope scope("native_batch_norm_backward", input);
  RowsView xv = rows_view(input);
  const int C = (int)xv.C;
  const int vec = input.scalar_type() == at::kFloat ? 4 : 8;
  TORCH_CHECK(C % vec == 0, "b200 batch_norm_backward: channels must be a multiple of ", vec);
  // grad in the same memory layout as x
  Tensor dy = at::empty_strided(xv.t.sizes(), xv.t.strides(), grad_out.options());
  if (grad_out.sizes() == xv.t.sizes() && grad_out.strides() == xv.t.strides()) dy = grad_out;
  else dy.copy_(grad_out);
  auto fopt = input.options().dtype(at::kFloat);
  Tensor wk;
  const void* gamma = opt_ptr(weight, wk);
  const int pdt = gamma ? to_b200_dtype(wk.scalar_type()) : B200_F32;
  const int xdt = to_b200_dtype(input.scalar_type());
  Tensor mean_t, invstd_t;
  int mdt = B200_F32;
  if (train) {
    TORCH_CHECK(save_mean.has_value() && save_mean->defined() && save_invstd.has_value() && save_invstd->defined(),
                "batch_norm_backward: saved statistics missing");
    mean_t = save_mean->contiguous();
    invstd_t = save_invstd->to(at::kFloat).contiguous();
    mdt = to_b200_dtype(mean_t.scalar_type());
  } else {
    mean_t = running_mean->contiguous();
    mdt = to_b200_dtype(mean_t.scalar_type());
    invstd_t = at::empty({C}, fopt);
    Tensor rv = running_var->contiguous();
    B200_KERNEL_CHECK(b200_bn_invstd_from_var(rv.data_ptr(), to_b200_dtype(rv.scalar_type()), C, (float)eps,
                                              invstd_t.data_ptr<float>(), scope.stream()));
  }
  Tensor dx, dgamma, dbeta;
  if (mask[0]) dx = at::empty_strided(xv.t.sizes(), xv.t.strides(), input.options());
  if (mask[1]) dgamma = at::empty({C}, fopt);
  if (mask[2]) dbeta = at::empty({C}, fopt);
  if (input.numel() == 0) {
    if (dgamma.defined()) dgamma.zero_();
    if (dbeta.defined()) dbeta.zero_();
    return {dx, dgamma, dbeta};
  }
  Tensor sums = at::zeros({2 * C}, input.options().dtype(at::kDouble));
  B200_KERNEL_CHECK(b200_bn_backward_reduce(dy.data_ptr(), xdt, xv.t.data_ptr(), xdt, mean_t.data_ptr(), mdt,
                                            invstd_t.data_ptr<float>(), nullptr, 0, xv.rows, C,
                                            sums.data_ptr<double>(), scope.stream()));
  B200_KERNEL_CHECK(b200_bn_backward_apply(dy.data_ptr(), xdt, xv.t.data_ptr(), xdt, mean_t.data_ptr(), mdt,
                                           invstd_t.data_ptr<float>(), gamma, pdt, nullptr, 0, sums.data_ptr<double>(),
                                           xv.rows, C, train ? 1 : 0, dx.defined() ? dx.data_ptr() : nullptr, xdt,
                                           dgamma.defined() ? dgamma.data_ptr<float>() : nullptr,
                                           dbeta.defined() ? dbeta.data_ptr<float>() : nullptr, nullptr, scope.stream()));
  if (weight.has_value() && weight->defined() && weight->scalar_type() != at::kFloat) {
    if (dgamma.defined()) dgamma = dgamma.to(weight->scalar_type());
    if (dbeta.defined()) dbeta = dbeta.to(weight->scalar_type());
  }
  return {in_format_of(dx, input), dgamma, dbeta};
}

std::tuple<Tensor, Tensor, Tensor> k_native_batch_norm_backward(
    const Tensor& grad_out, const Tensor& input, const std::optional<Tensor>& weight,
    const std::optional<Tensor>& running_mean, const std::optional<Tensor>& running_var,
    const std::optional<Tensor>& save_mean, const std::optional<Tensor>& save_invstd, bool train, double eps,
    std::array<bool, 3> mask) {
  return B200_DISPATCH("native_batch_norm_backward",
                       batch_norm_backward_device(grad_out, input, weight, running_mean, running_var, save_mean,
                                                  save_invstd, train, eps, mask),
                       B200_CPU(native_batch_norm_backward, grad_out, input, weight, running_mean, running_var,
                                save_mean, save_invstd, train, eps, mask));
}


// ---------------------------------------------------------------- fused BN + act
// out = act(batch_norm(x) + residual); act 1 = ReLU.  Training statistics and running
// statistics behave exactly like native_batch_norm.  The backward masks the incoming
// gradient with out > 0 inside the reduction and apply kernels, so neither the ReLU nor
// the residual add costs a pass over the activation.
}  // namespace

namespace {
// Zeroed fp64 scratch (2 x 8192 channel sums) and a zeroed counter word per (device, queue).  Contract: whoever
// takes it finds it cleared and leaves it cleared (b200_bn_backward_apply2 does the clearing on the device).
struct BnScratch {
  at::Tensor sums, counter;
};
std::mutex g_bn_scratch_mu;
std::map<std::pair<int, void*>, BnScratch> g_bn_scratch;
const bool g_bn_scratch_dropper = [] {
  registerCacheDropper([] {
    std::lock_guard<std::mutex> lk(g_bn_scratch_mu);
    g_bn_scratch.clear();
  });
  return true;
}();
BnScratch* bn_scratch(int device, void* stream) {
  std::lock_guard<std::mutex> lk(g_bn_scratch_mu);
  auto key = std::make_pair(device, stream);
  auto it = g_bn_scratch.find(key);
  if (it == g_bn_scratch.end()) {
    auto opt = at::TensorOptions().device(c10::Device(c10::DeviceType::PrivateUse1, device));
    BnScratch sc{at::zeros({2 * 8192}, opt.dtype(at::kDouble)), at::zeros({1}, opt.dtype(at::kInt))};
    it = g_bn_scratch.emplace(key, std::move(sc)).first;
  }
  return &it->second;
}
void bn_scratch_drop(int device, void* stream) {
  std::lock_guard<std::mutex> lk(g_bn_scratch_mu);
  g_bn_scratch.erase(std::make_pair(device, stream));
}
}  // namespace

static std::tuple<at::Tensor, at::Tensor, at::Tensor> batch_norm_act_impl(const at::Tensor& input, const std::optional<at::Tensor>& weight,
                                                              const std::optional<at::Tensor>& bias,
                                                              const std::optional<at::Tensor>& running_mean,
                                                              const std::optional<at::Tensor>& running_var,
                                                              const std::optional<at::Tensor>& residual, bool training,
                                                              double momentum, double eps, int64_t act,
                                                              const std::optional<at::Tensor>& channel_sums,
                                                              at::Tensor* relu_mask, const at::Tensor* batch_counter = nullptr,
                                                              bool* counted = nullptr) {
  // batch_counter (num_batches_tracked): incremented by the fused kernel when that runs (*counted = true);
  // otherwise the caller adds one itself
  const bool has_res = residual.has_value() && residual->defined();
  auto compose = [&]() {
    auto r = at::native_batch_norm(input, weight, bias, running_mean, running_var, training, momentum, eps);
    at::Tensor y = std::get<0>(r);
    if (has_res) y = y + *residual;
    if (act == 1) y = at::relu(y);
    return std::make_tuple(y, std::get<1>(r), std::get<2>(r));
  };
  const int vec = input.scalar_type() == at::kFloat ? 4 : 8;
  if (use_cpu_path() || !is_b200(input) || !bn_dtype_ok(input.scalar_type()) || input.dim() < 2 || input.size(1) % vec != 0 ||
      input.numel() == 0 || (has_res && (residual->scalar_type() != input.scalar_type() || residual->sizes() != input.sizes())))
    return compose();
  OpScope scope("batch_norm_act", input);
  RowsView v = rows_view(input);
  const int C = (int)v.C;
  at::Tensor out = like_rows(v, input, input.scalar_type());
  at::Tensor res;
  if (has_res) {
    res = at::empty_strided(v.t.sizes(), v.t.strides(), residual->options());
    if (residual->sizes() == v.t.sizes() && residual->strides() == v.t.strides()) res = *residual;
    else res.copy_(*residual);
  }
  auto fopt = input.options().dtype(at::kFloat);
  at::Tensor wk, bk;
  const void* gamma = opt_ptr(weight, wk);
  const void* beta = opt_ptr(bias, bk);
  const int pdt = gamma ? to_b200_dtype(wk.scalar_type()) : (beta ? to_b200_dtype(bk.scalar_type()) : B200_F32);
  const int xdt = to_b200_dtype(input.scalar_type());
  at::Tensor save_mean, save_invstd;
  const void* mean_ptr;
  int mdt = B200_F32;
  at::Tensor rmk;
  if (training) {
    save_mean = at::empty({C}, fopt);
    save_invstd = at::empty({C}, fopt);
    // sums supplied by the producing convolution make the statistics pass unnecessary
    at::Tensor sums;
    if (channel_sums.has_value() && channel_sums->defined()) {
      TORCH_CHECK(is_b200(*channel_sums) && channel_sums->scalar_type() == at::kDouble && channel_sums->numel() == 2 * C &&
                      channel_sums->is_contiguous(),
                  "batch_norm_act: channel_sums must be a contiguous fp64 tensor of 2 * C elements on the device");
      sums = *channel_sums;
    } else {
      sums = at::zeros({2 * C}, input.options().dtype(at::kDouble));
      B200_KERNEL_CHECK(b200_bn_stats(v.t.data_ptr(), xdt, v.rows, C, sums.data_ptr<double>(), scope.stream()));
    }
    void* rm = nullptr;
    void* rv = nullptr;
    int rdt = B200_F32;
    if (running_mean.has_value() && running_mean->defined()) {
      rm = running_mean->data_ptr();
      rv = running_var->data_ptr();
      rdt = to_b200_dtype(running_mean->scalar_type());
    }
    // One launch: statistics from the sums, running-statistics update, normalisation (+ residual, ReLU, mask).
    void* fused_mask = nullptr;
    if (relu_mask && act == 1 && input.scalar_type() != at::kFloat && C % 8 == 0 && C <= 8192 && (v.rows * C) / 8 < 0xffffffffLL) {
      *relu_mask = at::empty({v.rows * C / 8}, input.options().dtype(at::kByte));
      fused_mask = relu_mask->data_ptr();
    }
    long long* counter_ptr = nullptr;
    if (batch_counter && batch_counter->defined() && is_b200(*batch_counter) && batch_counter->scalar_type() == at::kLong &&
        batch_counter->numel() == 1)
      counter_ptr = reinterpret_cast<long long*>(batch_counter->data_ptr());
    const int frc = b200_bn_apply_fused(v.t.data_ptr(), xdt, out.data_ptr(), v.rows, C, sums.data_ptr<double>(), (float)eps,
                                        (float)momentum, save_mean.data_ptr<float>(), save_invstd.data_ptr<float>(), rm, rv, rdt,
                                        gamma, beta, pdt, has_res ? res.data_ptr() : nullptr, (int)act, fused_mask, counter_ptr,
                                        scope.stream());
    if (frc == 0) {
      if (counted) *counted = counter_ptr != nullptr;
      note_kernel_launch();
      return {out, save_mean, save_invstd};
    }
    TORCH_CHECK(frc == 801, "b200 batch_norm_act: ", device_error_string(frc));
    if (relu_mask) *relu_mask = at::empty({0}, input.options().dtype(at::kByte));
    B200_KERNEL_CHECK(b200_bn_finalize(sums.data_ptr<double>(), v.rows, C, (float)eps, (float)momentum,
                                       save_mean.data_ptr<float>(), save_invstd.data_ptr<float>(), rm, rv, rdt, scope.stream()));
    mean_ptr = save_mean.data_ptr();
  } else {
    TORCH_CHECK(running_mean.has_value() && running_mean->defined(), "batch_norm_act: running statistics required in eval mode");
    save_mean = at::empty({0}, fopt);
    save_invstd = at::empty({C}, fopt);  // kept for the backward of frozen batch norm
    rmk = running_mean->contiguous();
    at::Tensor rv = running_var->contiguous();
    B200_KERNEL_CHECK(b200_bn_invstd_from_var(rv.data_ptr(), to_b200_dtype(rv.scalar_type()), C, (float)eps,
                                              save_invstd.data_ptr<float>(), scope.stream()));
    mean_ptr = rmk.data_ptr();
    mdt = to_b200_dtype(rmk.scalar_type());
  }
  void* mask_ptr = nullptr;
  if (relu_mask && act == 1 && input.scalar_type() != at::kFloat && C % 8 == 0 && C <= 8192 && (v.rows * C) / 8 < 0xffffffffLL) {
    // one bit per element of the ReLU output: what the backward needs instead of the output itself
    *relu_mask = at::empty({v.rows * C / 8}, input.options().dtype(at::kByte));
    mask_ptr = relu_mask->data_ptr();
  }
  B200_KERNEL_CHECK(b200_bn_apply_mask(v.t.data_ptr(), xdt, out.data_ptr(), xdt, v.rows, C, mean_ptr, mdt,
                                       save_invstd.data_ptr<float>(), gamma, beta, pdt, has_res ? res.data_ptr() : nullptr, xdt,
                                       (int)act, mask_ptr, scope.stream()));
  return {out, save_mean, save_invstd};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> batch_norm_act(const at::Tensor& input, const std::optional<at::Tensor>& weight,
                                                              const std::optional<at::Tensor>& bias,
                                                              const std::optional<at::Tensor>& running_mean,
                                                              const std::optional<at::Tensor>& running_var,
                                                              const std::optional<at::Tensor>& residual, bool training,
                                                              double momentum, double eps, int64_t act,
                                                              const std::optional<at::Tensor>& channel_sums) {
  check_same_device("batch_norm_act", input, weight, bias, running_mean, running_var, residual, channel_sums);
  return batch_norm_act_impl(input, weight, bias, running_mean, running_var, residual, training, momentum, eps, act, channel_sums,
                             nullptr);
}

// Same, plus a bit mask of the positive outputs (empty when the fast kernel does not apply): pass it to
// batch_norm_act_backward in place of the output.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> batch_norm_act_mask(
    const at::Tensor& input, const std::optional<at::Tensor>& weight, const std::optional<at::Tensor>& bias,
    const std::optional<at::Tensor>& running_mean, const std::optional<at::Tensor>& running_var,
    const std::optional<at::Tensor>& residual, bool training, double momentum, double eps, int64_t act,
    const std::optional<at::Tensor>& channel_sums, const std::optional<at::Tensor>& num_batches_tracked) {
  at::Tensor mask = at::empty({0}, input.options().dtype(at::kByte));
  const at::Tensor* nbt = (num_batches_tracked.has_value() && num_batches_tracked->defined()) ? &*num_batches_tracked : nullptr;
  bool counted = false;
  auto r = batch_norm_act_impl(input, weight, bias, running_mean, running_var, residual, training, momentum, eps, act, channel_sums,
                               &mask, nbt, &counted);
  if (nbt && !counted) const_cast<at::Tensor*>(nbt)->add_(1);
  return {std::get<0>(r), std::get<1>(r), std::get<2>(r), mask};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> batch_norm_act_backward(
    const at::Tensor& grad_out, const at::Tensor& out, const at::Tensor& input, const std::optional<at::Tensor>& weight,
    const std::optional<at::Tensor>& running_mean, const at::Tensor& save_mean, const at::Tensor& save_invstd, bool training,
    int64_t act, bool has_residual) {
  if (use_cpu_path()) {
    // Host path (host simulation, force-CPU mode): the same gradient from ordinary tensor operations.  The forward's
    // host path returns an empty mask, so `out` is the forward output here.
    TORCH_CHECK(out.scalar_type() != at::kByte, "batch_norm_act_backward (host path): expects the forward output, not a bit mask");
    TORCH_CHECK(save_invstd.numel() == input.size(1), "batch_norm_act_backward (host path): needs the saved inverse standard deviation");
    std::vector<int64_t> bshape(input.dim(), 1), rdims;
    bshape[1] = input.size(1);
    for (int64_t d = 0; d < input.dim(); ++d)
      if (d != 1) rdims.push_back(d);
    at::Tensor g = grad_out.to(at::kFloat);
    if (act == 1) g = g * out.gt(0).to(at::kFloat);
    at::Tensor dres = has_residual ? g.to(input.scalar_type()) : at::Tensor();
    const at::Tensor mean = training ? save_mean : *running_mean;
    at::Tensor invstd = save_invstd.to(at::kFloat).view(bshape);
    at::Tensor xhat = (input.to(at::kFloat) - mean.to(at::kFloat).view(bshape)) * invstd;
    at::Tensor dbeta = g.sum(rdims), dgamma = (g * xhat).sum(rdims);
    at::Tensor scale = invstd;
    if (weight.has_value() && weight->defined()) scale = scale * weight->to(at::kFloat).view(bshape);
    const double m = (double)(input.numel() / std::max<int64_t>(1, input.size(1)));
    at::Tensor dx = training ? scale * (g - dbeta.view(bshape) / m - xhat * (dgamma.view(bshape) / m)) : scale * g;
    return {dx.to(input.scalar_type()), dgamma, dbeta, dres};
  }
  TORCH_CHECK(is_b200(input), "batch_norm_act_backward: the input must be on the device");
  OpScope scope("batch_norm_act_backward", input);
  RowsView xv = rows_view(input);
  const int C = (int)xv.C;
  auto same_layout = [&](const at::Tensor& t) {
    if (t.sizes() == xv.t.sizes() && t.strides() == xv.t.strides()) return t;
    return at::empty_strided(xv.t.sizes(), xv.t.strides(), t.options()).copy_(t);
  };
  // `out` is either the forward output or, as a uint8 tensor, the bit mask of its positive elements
  const bool bitmask = out.scalar_type() == at::kByte && act == 1;
  at::Tensor dy = same_layout(grad_out), y = bitmask ? out.contiguous() : same_layout(out);
  auto fopt = input.options().dtype(at::kFloat);
  at::Tensor wk;
  const void* gamma = opt_ptr(weight, wk);
  const int pdt = gamma ? to_b200_dtype(wk.scalar_type()) : B200_F32;
  const int xdt = to_b200_dtype(input.scalar_type());
  at::Tensor mean_t = training ? save_mean.contiguous() : running_mean->contiguous();
  const int mdt = to_b200_dtype(mean_t.scalar_type());
  at::Tensor invstd = save_invstd.contiguous();
  at::Tensor dx = at::empty_strided(xv.t.sizes(), xv.t.strides(), input.options());
  at::Tensor dres = has_residual ? at::empty_strided(xv.t.sizes(), xv.t.strides(), input.options()) : at::Tensor();
  at::Tensor dgamma = at::empty({C}, fopt), dbeta = at::empty({C}, fopt);
  const void* mask = act == 1 ? y.data_ptr() : nullptr;
  const int mask_dt = bitmask ? (int)B200_U8 : xdt;
  if (bitmask) TORCH_CHECK(y.numel() * 8 == xv.rows * C, "batch_norm_act_backward: mask size does not match the input");
  // The fp64 sums live in a per-queue scratch buffer that the apply kernel clears after use, which saves a
  // memset launch per batch norm.  If anything throws in between, the buffer is dropped (it may be dirty).
  const bool vec_ok = C <= 8192 && C % (xdt == B200_F32 ? 4 : 8) == 0 && (xv.rows * C) / (xdt == B200_F32 ? 4 : 8) < 0xffffffffLL;
  BnScratch* scratch = vec_ok ? bn_scratch(input.device().index(), scope.stream()) : nullptr;
  at::Tensor sums = scratch ? scratch->sums : at::zeros({2 * C}, input.options().dtype(at::kDouble));
  try {
    B200_KERNEL_CHECK(b200_bn_backward_reduce(dy.data_ptr(), xdt, xv.t.data_ptr(), xdt, mean_t.data_ptr(), mdt,
                                              invstd.data_ptr<float>(), mask, mask_dt, xv.rows, C, sums.data_ptr<double>(),
                                              scope.stream()));
    B200_KERNEL_CHECK(b200_bn_backward_apply2(dy.data_ptr(), xdt, xv.t.data_ptr(), xdt, mean_t.data_ptr(), mdt,
                                              invstd.data_ptr<float>(), gamma, pdt, mask, mask_dt, sums.data_ptr<double>(), xv.rows, C,
                                              training ? 1 : 0, dx.data_ptr(), xdt, dgamma.data_ptr<float>(),
                                              dbeta.data_ptr<float>(), has_residual ? dres.data_ptr() : nullptr,
                                              scratch ? reinterpret_cast<unsigned*>(scratch->counter.data_ptr()) : nullptr,
                                              scope.stream()));
  } catch (...) {
    if (scratch) bn_scratch_drop(input.device().index(), scope.stream());
    throw;
  }
  if (weight.has_value() && weight->defined() && weight->scalar_type() != at::kFloat) {
    dgamma = dgamma.to(weight->scalar_type());
    dbeta = dbeta.to(weight->scalar_type());
  }
  return {dx, dgamma, dbeta, dres};
}

namespace {
// ------------------------------------------------------------------- layer norm
std::tuple<Tensor, Tensor, Tensor> layer_norm_device(const Tensor& input, at::IntArrayRef normalized_shape,
                                                     const std::optional<Tensor>& weight,
                                                     const std::optional<Tensor>& bias, double eps) {
  TORCH_CHECK(bn_dtype_ok(input.scalar_type()), "b200 layer_norm: unsupported dtype ", input.scalar_type());
  OpScope scope("native_layer_norm", input);
  int64_t cols = 1;
  for (auto s : normalized_shape) cols *= s;
  const int64_t rows = cols ? input.numel() / cols : 0;
  Tensor x = input.contiguous();
  Tensor y = at::empty_like(x);
  std::vector<int64_t> stat_shape(input.sizes().begin(), input.sizes().end() - normalized_shape.size());
  for (size_t i = 0; i < normalized_shape.size(); ++i) stat_shape.push_back(1);
  auto fopt = input.options().dtype(at::kFloat);
  Tensor mean = at::empty(stat_shape, fopt), rstd = at::empty(stat_shape, fopt);
  Tensor wk, bk;
  const void* gamma = opt_ptr(weight, wk);
  const void* beta = opt_ptr(bias, bk);
  const int pdt = gamma ? to_b200_dtype(wk.scalar_type()) : (beta ? to_b200_dtype(bk.scalar_type()) : B200_F32);
  B200_KERNEL_CHECK(b200_layernorm_fwd(x.data_ptr(), to_b200_dtype(x.scalar_type()), rows, (int)cols, gamma, beta, pdt,
                                       (float)eps, y.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                                       scope.stream()));
  if (input.scalar_type() != at::kFloat) {
    // stock kernels return statistics in the input dtype
    return {y, mean.to(input.scalar_type()), rstd.to(input.scalar_type())};
  }
  return {y, mean, rstd};
}
std::tuple<Tensor, Tensor, Tensor> k_native_layer_norm(const Tensor& input, at::IntArrayRef normalized_shape,
                                                     const std::optional<Tensor>& weight,
                                                     const std::optional<Tensor>& bias, double eps) {
  check_same_device("layer_norm", input, weight, bias);
  return B200_DISPATCH("native_layer_norm", layer_norm_device(input, normalized_shape, weight, bias, eps),
                       B200_CPU(native_layer_norm, input, normalized_shape, weight, bias, eps));
}

std::tuple<Tensor, Tensor, Tensor> layer_norm_backward_device(const Tensor& grad_out, const Tensor& input,
                                                              at::IntArrayRef normalized_shape, const Tensor& mean,
                                                              const Tensor& rstd, const std::optional<Tensor>& weight,
                                                              const std::optional<Tensor>& bias,
                                                              std::array<bool, 3> mask) {
  TORCH_CHECK(bn_dtype_ok(input.scalar_type()) && grad_out.scalar_type() == input.scalar_type(),
              "b200 layer_norm_backward: unsupported dtypes");
  OpScope scope("native_layer_norm_backward", input);
  int64_t cols = 1;
  for (auto s : normalized_shape) cols *= s;
  const int64_t rows = cols ? input.numel() / cols : 0;
  Tensor x = input.contiguous(), dy = grad_out.contiguous();
  Tensor m = mean.to(at::kFloat).contiguous(), r = rstd.to(at::kFloat).contiguous();
  Tensor wk;
  const void* gamma = opt_ptr(weight, wk);
  const int pdt = gamma ? to_b200_dtype(wk.scalar_type()) : B200_F32;
  Tensor dx, dg, db;
  auto fopt = input.options().dtype(at::kFloat);
  if (mask[0]) dx = at::empty_like(x);
  if (mask[1]) dg = at::zeros({cols}, fopt);
  if (mask[2]) db = at::zeros({cols}, fopt);
  B200_KERNEL_CHECK(b200_layernorm_bwd(dy.data_ptr(), x.data_ptr(), to_b200_dtype(x.scalar_type()), rows, (int)cols,
                                       gamma, pdt, m.data_ptr<float>(), r.data_ptr<float>(),
                                       dx.defined() ? dx.data_ptr() : nullptr, dg.defined() ? dg.data_ptr<float>() : nullptr,
                                       db.defined() ? db.data_ptr<float>() : nullptr, scope.stream()));
  if (dg.defined() && weight.has_value() && weight->defined()) dg = dg.to(weight->scalar_type()).view(weight->sizes());
  if (db.defined() && bias.has_value() && bias->defined()) db = db.to(bias->scalar_type()).view(bias->sizes());
  else if (db.defined() && weight.has_value() && weight->defined()) db = db.to(weight->scalar_type()).view(weight->sizes());
  return {dx, dg, db};
}
std::tuple<Tensor, Tensor, Tensor> k_native_layer_norm_backward(const Tensor& grad_out, const Tensor& input,
                                                              at::IntArrayRef normalized_shape, const Tensor& mean,
                                                              const Tensor& rstd, const std::optional<Tensor>& weight,
                                                              const std::optional<Tensor>& bias,
                                                              std::array<bool, 3> mask) {
  return B200_DISPATCH("native_layer_norm_backward",
                       layer_norm_backward_device(grad_out, input, normalized_shape, mean, rstd, weight, bias, mask),
                       B200_CPU(native_layer_norm_backward, grad_out, input, normalized_shape, mean, rstd, weight, bias, mask));
}

}  // namespace

// The batch-norm forwards are registered under host simulation too: their host path is the one above, not the boxed
// fallback (see there).
TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("native_batch_norm", TORCH_FN(k_native_batch_norm));
  m.impl("_native_batch_norm_legit", TORCH_FN(bn_legit));
  m.impl("_native_batch_norm_legit.no_stats", TORCH_FN(bn_legit_no_stats));
  m.impl("_native_batch_norm_legit_no_training", TORCH_FN(bn_legit_no_training));
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("native_batch_norm_backward", TORCH_FN(k_native_batch_norm_backward));
  m.impl("native_layer_norm", TORCH_FN(k_native_layer_norm));
  m.impl("native_layer_norm_backward", TORCH_FN(k_native_layer_norm_backward));
}

}  // namespace ops
}  // namespace catch_b200
