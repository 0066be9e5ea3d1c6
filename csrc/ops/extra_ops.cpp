// Operators that the reference runs on the device and that are built here from this backend's own
// kernels: _unique2 (torch_mlu/csrc/aten/operators/cnnl/unique.cpp:37), index_fill_ (index_fill.cpp:37),
// nll_loss2d forward / backward (nllloss.cpp:87, nllloss_backward.cpp:68), linspace (linspace.cpp),
// equal (logic.cpp:269), plus cumsum over integers, which the unique kernel chain needs anyway.
#include <cstring>

#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

// ---- cumsum (integral and bool inputs, int64 result; the int64 scan kernel) -------------------------
Tensor scan_i64(const Tensor& flat_i64, const OpScope& scope) {
  Tensor out = at::empty_like(flat_i64);
  const int64_t n = flat_i64.numel();
  if (n == 0) return out;
  Workspace ws((size_t)b200_scan_workspace_elems(n) * 8, scope);
  B200_KERNEL_CHECK(b200_inclusive_scan_i64(i64ptr(flat_i64), i64ptr(out), n, ws.as<long long>(), scope.stream()));
  return out;
}
Tensor cumsum_device(const Tensor& self, int64_t dim, std::optional<at::ScalarType> dtype) {
  const auto out_t = dtype.value_or(c10::isIntegralType(self.scalar_type(), true) ? at::kLong : self.scalar_type());
  TORCH_CHECK(c10::isIntegralType(self.scalar_type(), true) && out_t == at::kLong && self.dim() <= 1,
              "b200 cumsum: only 1-D integral inputs with an int64 result have a device kernel");
  OpScope scope("cumsum", self);
  Tensor x = self.reshape({-1}).to(at::kLong).contiguous();
  return scan_i64(x, scope).view(self.sizes());
}
Tensor k_cumsum(const Tensor& self, int64_t dim, std::optional<at::ScalarType> dtype) {
  return B200_DISPATCH("cumsum", cumsum_device(self, dim, dtype), B200_CPU(cumsum, self, dim, dtype));
}

// ---- _unique2: sort, mark the first element of every run, scan the marks -----------------------------
std::tuple<Tensor, Tensor, Tensor> unique2_device(const Tensor& self, bool /*sorted*/, bool return_inverse, bool return_counts) {
  const auto t = self.scalar_type();
  TORCH_CHECK(to_b200_dtype(t) >= 0 && t != at::kComplexFloat && t != at::kComplexDouble, "b200 unique: unsupported dtype ", t);
  OpScope scope("_unique2", self);
  const int64_t n = self.numel();
  auto lopt = self.options().dtype(at::kLong);
  if (n == 0) return {at::empty({0}, self.options()), at::empty(self.sizes(), lopt), at::empty({0}, lopt)};
  Tensor flat = self.reshape({-1}).contiguous();
  Tensor sorted_vals = at::empty_like(flat), perm = at::empty({n}, lopt);
  {
    Workspace ws((size_t)b200_sort_long_workspace_bytes(1, n), scope);
    B200_KERNEL_CHECK(b200_sort_long(flat.data_ptr(), to_b200_dtype(t), (int)flat.element_size(), 1, n, 0, n, sorted_vals.data_ptr(),
                                     i64ptr(perm), ws.get(), scope.stream()));
  }
  // first[i] = 1 where a new run starts (element 0 always does)
  Tensor first = at::ones({n}, lopt);
  if (n > 1) first.narrow(0, 1, n - 1).copy_(at::ne(sorted_vals.narrow(0, 1, n - 1), sorted_vals.narrow(0, 0, n - 1)));
  Tensor run_id = scan_i64(first, scope).sub_(1);            // unique index of every sorted element
  Tensor first_b = first.to(at::kBool);
  Tensor values = sorted_vals.masked_select(first_b);          // host sync: the number of unique values
  Tensor inverse = at::empty({0}, lopt), counts = at::empty({0}, lopt);
  if (return_inverse) {
    inverse = at::empty({n}, lopt);
    inverse.index_put_({perm}, run_id);
    inverse = inverse.view(self.sizes());
  }
  if (return_counts) {
    Tensor starts = at::nonzero(first_b).reshape({-1});
    Tensor ends = at::cat({starts.narrow(0, 1, starts.numel() - 1), at::full({1}, n, lopt)});
    counts = ends - starts;
  }
  return {values, inverse, counts};
}
std::tuple<Tensor, Tensor, Tensor> k_unique2(const Tensor& self, bool sorted, bool return_inverse, bool return_counts) {
  return B200_DISPATCH("_unique2", unique2_device(self, sorted, return_inverse, return_counts),
                       B200_CPU(_unique2, self, sorted, return_inverse, return_counts));
}

// ---- index_fill_ ---------------------------------------------------------------------------------------
Tensor bad_flag_tensor(const Tensor& like) { return at::zeros({1}, like.options().dtype(at::kInt)); }

Tensor& index_fill_device(Tensor& self, int64_t dim, const Tensor& index, const at::Scalar& value) {
  TORCH_CHECK(index.scalar_type() == at::kLong || index.scalar_type() == at::kInt, "index_fill_: index must be int32 or int64");
  TORCH_CHECK(index.dim() <= 1, "index_fill_: index must be a vector or a scalar");
  const int es = (int)self.element_size();
  TORCH_CHECK(es <= 8 && !self.is_complex(), "b200 index_fill_: unsupported dtype ", self.scalar_type());
  OpScope scope("index_fill_", self);
  if (self.numel() == 0 || index.numel() == 0) return self;
  Tensor x = self.dim() == 0 ? self.unsqueeze(0) : self;
  dim = at::maybe_wrap_dim(dim, x.dim());
  // the kernel works on [outer][n][inner]: a contiguous tensor is used in place, anything else through a dense copy
  Tensor work = x.is_contiguous() ? x : x.contiguous();
  int64_t outer = 1, inner = 1;
  for (int64_t d = 0; d < dim; ++d) outer *= work.size(d);
  for (int64_t d = dim + 1; d < work.dim(); ++d) inner *= work.size(d);
  Tensor idx = index.to(at::kLong).reshape({-1}).contiguous();
  // the value's bit pattern in the tensor's dtype
  Tensor host = at::empty({1}, at::TensorOptions().dtype(self.scalar_type())).fill_(value);
  unsigned long long bits = 0;
  std::memcpy(&bits, host.data_ptr(), es);
  Tensor bad = bad_flag_tensor(self);
  B200_KERNEL_CHECK(b200_index_fill(work.data_ptr(), es, i64ptr(idx), outer, work.size(dim), idx.numel(), inner, bits,
                                    bad.data_ptr<int>(), scope.stream()));
  if (flags().async_disable) TORCH_CHECK(bad.item<int>() == 0, "index_fill_: index out of range");
  if (!work.is_same(x)) x.copy_(work);
  return self;
}
Tensor& k_index_fill_scalar(Tensor& self, int64_t dim, const Tensor& index, const at::Scalar& value) {
  B200_DISPATCH("index_fill_.int_Scalar", (void)index_fill_device(self, dim, index, value),
                (void)B200_CPU(index_fill__int_Scalar, self, dim, index, value));
  return self;
}
Tensor& k_index_fill_tensor(Tensor& self, int64_t dim, const Tensor& index, const Tensor& value) {
  TORCH_CHECK(value.dim() == 0, "index_fill_ only supports a 0-dimensional value tensor");
  return k_index_fill_scalar(self, dim, index, value.item());
}
Tensor k_index_fill_scalar_f(const Tensor& self, int64_t dim, const Tensor& index, const at::Scalar& value) {
  Tensor out = self.clone(at::MemoryFormat::Contiguous);
  return k_index_fill_scalar(out, dim, index, value);
}

// ---- nll_loss2d: the row kernels on an NHWC view of the class scores -----------------------------------
std::tuple<Tensor, Tensor> nll2d_fwd_device(const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight,
                                            int64_t reduction, int64_t ignore_index) {
  TORCH_CHECK(self.dim() == 4 && target.dim() == 3, "b200 nll_loss2d: expects [N, C, H, W] scores and [N, H, W] targets");
  const int64_t N = self.size(0), C = self.size(1), H = self.size(2), W = self.size(3);
  Tensor rows = self.permute({0, 2, 3, 1}).reshape({N * H * W, C});
  auto r = at::nll_loss_forward(rows, target.reshape({-1}), weight, reduction, ignore_index);
  Tensor out = std::get<0>(r);
  if (reduction == at::Reduction::None) out = out.view({N, H, W});
  return {out, std::get<1>(r)};
}
std::tuple<Tensor, Tensor> k_nll_loss2d_forward(const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight,
                                                int64_t reduction, c10::SymInt ignore_index) {
  const int64_t ig = ignore_index.expect_int();
  check_same_device("nll_loss2d", self, target, weight);
  return B200_DISPATCH("nll_loss2d_forward", nll2d_fwd_device(self, target, weight, reduction, ig),
                       B200_CPU_SYMINT(nll_loss2d_forward, self, target, weight, reduction, ignore_index));
}
Tensor nll2d_bwd_device(const Tensor& grad, const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight,
                        int64_t reduction, int64_t ignore_index, const Tensor& total_weight) {
  TORCH_CHECK(self.dim() == 4 && target.dim() == 3, "b200 nll_loss2d_backward: expects [N, C, H, W] scores and [N, H, W] targets");
  const int64_t N = self.size(0), C = self.size(1), H = self.size(2), W = self.size(3);
  Tensor rows = self.permute({0, 2, 3, 1}).reshape({N * H * W, C});
  Tensor g = reduction == at::Reduction::None ? grad.reshape({-1}) : grad;
  Tensor drows = at::nll_loss_backward(g, rows, target.reshape({-1}), weight, reduction, ignore_index, total_weight);
  // [N*H*W, C] is the channels-last memory of the [N, C, H, W] gradient
  return drows.view({N, H, W, C}).permute({0, 3, 1, 2});
}
Tensor k_nll_loss2d_backward(const Tensor& grad, const Tensor& self, const Tensor& target, const std::optional<Tensor>& weight,
                             int64_t reduction, c10::SymInt ignore_index, const Tensor& total_weight) {
  const int64_t ig = ignore_index.expect_int();
  return B200_DISPATCH("nll_loss2d_backward", nll2d_bwd_device(grad, self, target, weight, reduction, ig, total_weight),
                       B200_CPU_SYMINT(nll_loss2d_backward, grad, self, target, weight, reduction, ignore_index, total_weight));
}

// ---- linspace: out[i] = start + i * step, the upper half counted down from `end` (as the stock kernels do,
// so that both ends are exact) -----------------------------------------------------------------------------
Tensor& linspace_out_device(const at::Scalar& start, const at::Scalar& end, int64_t steps, Tensor& out) {
  TORCH_CHECK(steps >= 0, "number of steps must be non-negative");
  const auto t = out.scalar_type();
  TORCH_CHECK(t == at::kFloat || t == at::kBFloat16 || t == at::kHalf || t == at::kDouble || t == at::kLong || t == at::kInt,
              "b200 linspace: unsupported dtype ", t);
  if (out.numel() != steps) out.resize_({steps});
  if (steps == 0) return out;
  OpScope scope("linspace", out);
  Tensor dst = out.is_contiguous() ? out : at::empty({steps}, out.options());
  const double s = start.toDouble(), e = end.toDouble();
  if (steps == 1) {
    dst.fill_(start);
  } else {
    const double step = (e - s) / (double)(steps - 1);
    const int64_t half = steps / 2;
    if (half > 0) B200_KERNEL_CHECK(b200_arange(dst.data_ptr(), to_b200_dtype(t), half, s, step, scope.stream()));
    // elements half .. steps-1 are end - (steps-1-i) * step: an arange that starts at end - (steps-1-half)*step
    char* upper = static_cast<char*>(dst.data_ptr()) + half * dst.element_size();
    B200_KERNEL_CHECK(b200_arange(upper, to_b200_dtype(t), steps - half, e - step * (double)(steps - 1 - half), step, scope.stream()));
  }
  if (!dst.is_same(out)) out.copy_(dst);
  return out;
}
Tensor& k_linspace_out(const at::Scalar& start, const at::Scalar& end, int64_t steps, Tensor& out) {
  B200_DISPATCH("linspace.out", (void)linspace_out_device(start, end, steps, out), (void)B200_CPU(linspace_out, start, end, steps, out));
  return out;
}

// ---- equal --------------------------------------------------------------------------------------------
bool equal_device(const Tensor& self, const Tensor& other) {
  TORCH_CHECK(self.device() == other.device(), "equal: tensors must live on the same device");
  if (self.sizes() != other.sizes()) return false;
  if (self.numel() == 0) return true;
  if (self.scalar_type() != other.scalar_type()) return false;
  return !at::ne(self, other).any().item<bool>();
}
bool k_equal(const Tensor& self, const Tensor& other) {
  return B200_DISPATCH("equal", equal_device(self, other), B200_CPU(equal, self, other));
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("cumsum", TORCH_FN(k_cumsum));
  m.impl("_unique2", TORCH_FN(k_unique2));
  m.impl("index_fill_.int_Scalar", TORCH_FN(k_index_fill_scalar));
  m.impl("index_fill_.int_Tensor", TORCH_FN(k_index_fill_tensor));
  m.impl("index_fill.int_Scalar", TORCH_FN(k_index_fill_scalar_f));
  m.impl("nll_loss2d_forward", TORCH_FN(k_nll_loss2d_forward));
  m.impl("nll_loss2d_backward", TORCH_FN(k_nll_loss2d_backward));
  m.impl("linspace.out", TORCH_FN(k_linspace_out));
  m.impl("equal", TORCH_FN(k_equal));
}

}  // namespace ops
}  // namespace catch_b200
