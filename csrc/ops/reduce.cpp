// Reduction operators: sum / mean / prod / amax / amin / max / min (with
// indices) / any / all / norm / argmax / argmin.
//
// Parity: torch_mlu/csrc/aten/operators/cnnl/reduceOps.cpp:122-480.  Differences
// on purpose: `dtype=` is honoured, half / bf16 accumulate in fp32, and integer or
// fp64 inputs take the CPU path instead of being computed in fp32.
#include <ATen/WrapDimUtilsMulti.h>
#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

bool f_ok(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf; }

std::vector<int64_t> out_shape(const Tensor& x, const std::bitset<64>& mask, bool keepdim) {
  std::vector<int64_t> s;
  for (int64_t d = 0; d < x.dim(); ++d) {
    if (mask[d]) { if (keepdim) s.push_back(1); }
    else s.push_back(x.size(d));
  }
  return s;
}

// Core: reduce `x` over the dims in `mask` into a fresh contiguous tensor.
Tensor reduce_core(const Tensor& x, std::bitset<64> mask, bool keepdim, int op, at::ScalarType out_dtype,
                   Tensor* indices) {
  OpScope scope("reduce", x);
  B200ReduceParams p;
  std::memset(&p, 0, sizeof(p));
  p.op = op;
  p.in_dtype = to_b200_dtype(x.scalar_type());
  p.out_dtype = to_b200_dtype(out_dtype);
  p.n_out = 1; p.n_red = 1;
  for (int64_t d = 0; d < x.dim(); ++d) {
    if (x.size(d) == 1) continue;
    if (mask[d]) {
      // merge with the previous reduced dim when contiguous in memory
      if (p.n_reduced > 0 && p.red_in_stride[p.n_reduced - 1] == x.stride(d) * x.size(d) && mask[d - 1]) {
        p.red_size[p.n_reduced - 1] *= x.size(d);
        p.red_in_stride[p.n_reduced - 1] = x.stride(d);
      } else {
        TORCH_CHECK(p.n_reduced < B200_RED_MAX_DIMS, "b200 reduce: too many reduced dimensions");
        p.red_size[p.n_reduced] = x.size(d);
        p.red_in_stride[p.n_reduced++] = x.stride(d);
      }
      p.n_red *= x.size(d);
    } else {
      TORCH_CHECK(p.n_kept < B200_RED_MAX_DIMS, "b200 reduce: too many kept dimensions");
      p.kept_size[p.n_kept] = x.size(d);
      p.kept_in_stride[p.n_kept++] = x.stride(d);
      p.n_out *= x.size(d);
    }
  }
  Tensor out = empty_b200(out_shape(x, mask, keepdim), out_dtype, x.device().index());
  if (indices) *indices = empty_b200(out_shape(x, mask, keepdim), at::kLong, x.device().index());
  if (out.numel() == 0) return out;
  p.in = x.data_ptr();
  p.out = out.data_ptr();
  p.out_index = indices ? i64ptr(*indices) : nullptr;
  const int ws = b200_reduce_plan(&p);
  Workspace w((size_t)ws * sizeof(float), scope);
  p.workspace = w.as<float>();
  B200_KERNEL_CHECK(b200_reduce(&p, scope.stream()));
  return out;
}

std::bitset<64> make_mask(at::OptionalIntArrayRef dims, int64_t ndim) {
  std::bitset<64> m;
  if (!dims.has_value() || dims->empty()) {
    for (int64_t d = 0; d < ndim; ++d) m.set(d);
    return m;
  }
  return at::dim_list_to_bitset(*dims, ndim);
}

Tensor sum_like(const Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype, int op) {
  const at::ScalarType odt = dtype.value_or(self.scalar_type());
  TORCH_CHECK(f_ok(self.scalar_type()) && f_ok(odt), "b200 reduce: dtype ", self.scalar_type(), " -> ", odt, " runs on the CPU path");
  TORCH_CHECK(self.numel() > 0 || op == RED_SUM, "b200 reduce: empty input");
  if (self.numel() == 0) return at::zeros(out_shape(self, make_mask(dim, self.dim()), keepdim), self.options().dtype(odt));
  return reduce_core(self, make_mask(dim, self.dim()), keepdim, op, odt, nullptr);
}

Tensor k_sum_dim(const Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype) {
  return B200_DISPATCH("sum", sum_like(self, dim, keepdim, dtype, RED_SUM), B200_CPU(sum_dim_IntList, self, dim, keepdim, dtype));
}
Tensor k_mean_dim(const Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, std::optional<at::ScalarType> dtype) {
  return B200_DISPATCH("mean", sum_like(self, dim, keepdim, dtype, RED_MEAN), B200_CPU(mean_dim, self, dim, keepdim, dtype));
}
Tensor k_prod_dim(const Tensor& self, int64_t dim, bool keepdim, std::optional<at::ScalarType> dtype) {
  const int64_t d[1] = {dim};
  return B200_DISPATCH("prod", sum_like(self, at::IntArrayRef(d, 1), keepdim, dtype, RED_PROD),
                       B200_CPU(prod_dim_int, self, dim, keepdim, dtype));
}
Tensor k_amax(const Tensor& self, at::IntArrayRef dim, bool keepdim) {
  return B200_DISPATCH("amax", sum_like(self, dim, keepdim, std::nullopt, RED_MAX), B200_CPU(amax, self, dim, keepdim));
}
Tensor k_amin(const Tensor& self, at::IntArrayRef dim, bool keepdim) {
  return B200_DISPATCH("amin", sum_like(self, dim, keepdim, std::nullopt, RED_MIN), B200_CPU(amin, self, dim, keepdim));
}
Tensor k_max_all(const Tensor& self) {
  return B200_DISPATCH("max", sum_like(self, std::nullopt, false, std::nullopt, RED_MAX), B200_CPU(max, self));
}
Tensor k_min_all(const Tensor& self) {
  return B200_DISPATCH("min", sum_like(self, std::nullopt, false, std::nullopt, RED_MIN), B200_CPU(min, self));
}
std::tuple<Tensor, Tensor> minmax_dim(const Tensor& self, int64_t dim, bool keepdim, int op) {
  TORCH_CHECK(f_ok(self.scalar_type()) && self.numel() > 0, "b200 max/min: runs on the CPU path");
  dim = at::maybe_wrap_dim(dim, self.dim());
  std::bitset<64> m;
  if (self.dim() > 0) m.set(dim);
  Tensor idx;
  Tensor v = reduce_core(self, m, keepdim, op, self.scalar_type(), &idx);
  return {v, idx};
}
std::tuple<Tensor, Tensor> k_max_dim(const Tensor& self, int64_t dim, bool keepdim) {
  return B200_DISPATCH("max.dim", minmax_dim(self, dim, keepdim, RED_MAX), B200_CPU(max_dim, self, dim, keepdim));
}
std::tuple<Tensor, Tensor> k_min_dim(const Tensor& self, int64_t dim, bool keepdim) {
  return B200_DISPATCH("min.dim", minmax_dim(self, dim, keepdim, RED_MIN), B200_CPU(min_dim, self, dim, keepdim));
}
Tensor arg_impl(const Tensor& self, std::optional<int64_t> dim, bool keepdim, int op) {
  TORCH_CHECK(f_ok(self.scalar_type()) && self.numel() > 0, "b200 argmax/argmin: runs on the CPU path");
  if (!dim.has_value()) {
    Tensor flat = self.contiguous().view({-1});
    std::bitset<64> m;
    m.set(0);
    return reduce_core(flat, m, false, op, at::kLong, nullptr);
  }
  std::bitset<64> m;
  if (self.dim() > 0) m.set(at::maybe_wrap_dim(*dim, self.dim()));
  return reduce_core(self, m, keepdim, op, at::kLong, nullptr);
}
Tensor k_argmax(const Tensor& self, std::optional<int64_t> dim, bool keepdim) {
  return B200_DISPATCH("argmax", arg_impl(self, dim, keepdim, RED_ARGMAX), B200_CPU(argmax, self, dim, keepdim));
}
Tensor k_argmin(const Tensor& self, std::optional<int64_t> dim, bool keepdim) {
  return B200_DISPATCH("argmin", arg_impl(self, dim, keepdim, RED_ARGMIN), B200_CPU(argmin, self, dim, keepdim));
}
Tensor norm_impl(const Tensor& self, const std::optional<at::Scalar>& p, at::IntArrayRef dim, bool keepdim,
                 std::optional<at::ScalarType> dtype) {
  const double pv = p.has_value() ? p->toDouble() : 2.0;
  int op;
  if (pv == 2.0) op = RED_NORM2;
  else if (pv == 1.0) op = RED_NORM1;
  else if (std::isinf(pv) && pv > 0) op = RED_NORM_INF;
  else TORCH_CHECK(false, "b200 norm: only p = 1, 2 and inf have device kernels");
  return sum_like(self, dim, keepdim, dtype, op);
}
Tensor k_norm_dim(const Tensor& self, const std::optional<at::Scalar>& p, at::IntArrayRef dim, bool keepdim) {
  return B200_DISPATCH("norm", norm_impl(self, p, dim, keepdim, std::nullopt), B200_CPU(norm_ScalarOpt_dim, self, p, dim, keepdim));
}
Tensor k_linalg_vector_norm(const Tensor& self, const at::Scalar& ord, at::OptionalIntArrayRef dim, bool keepdim,
                            std::optional<at::ScalarType> dtype) {
  return B200_DISPATCH("linalg_vector_norm",
                       norm_impl(self, ord, dim.has_value() ? *dim : at::IntArrayRef(), keepdim, dtype),
                       B200_CPU(linalg_vector_norm, self, ord, dim, keepdim, dtype));
}
Tensor anyall(const Tensor& self, int op) {
  TORCH_CHECK(self.numel() > 0, "b200 any/all: empty input runs on the CPU path");
  std::bitset<64> m;
  for (int64_t d = 0; d < self.dim(); ++d) m.set(d);
  return reduce_core(self, m, false, op, at::kBool, nullptr);
}
Tensor anyall_dim(const Tensor& self, int64_t dim, bool keepdim, int op) {
  TORCH_CHECK(self.numel() > 0, "b200 any/all: empty input runs on the CPU path");
  std::bitset<64> m;
  if (self.dim() > 0) m.set(at::maybe_wrap_dim(dim, self.dim()));
  return reduce_core(self, m, keepdim, op, at::kBool, nullptr);
}
Tensor k_any_dim(const Tensor& self, int64_t dim, bool keepdim) {
  return B200_DISPATCH("any.dim", anyall_dim(self, dim, keepdim, RED_ANY), B200_CPU(any_dim, self, dim, keepdim));
}
Tensor k_all_dim(const Tensor& self, int64_t dim, bool keepdim) {
  return B200_DISPATCH("all.dim", anyall_dim(self, dim, keepdim, RED_ALL), B200_CPU(all_dim, self, dim, keepdim));
}
Tensor k_prod_all(const Tensor& self, std::optional<at::ScalarType> dtype) {
  return B200_DISPATCH("prod", sum_like(self, std::nullopt, false, dtype, RED_PROD), B200_CPU(prod, self, dtype));
}
Tensor k_norm_dim_dtype(const Tensor& self, const std::optional<at::Scalar>& p, at::IntArrayRef dim, bool keepdim,
                        at::ScalarType dtype) {
  return B200_DISPATCH("norm", norm_impl(self, p, dim, keepdim, dtype),
                       B200_CPU(norm_ScalarOpt_dim_dtype, self, p, dim, keepdim, dtype));
}
Tensor k_any(const Tensor& self) { return B200_DISPATCH("any", anyall(self, RED_ANY), B200_CPU(any, self)); }
Tensor k_all(const Tensor& self) { return B200_DISPATCH("all", anyall(self, RED_ALL), B200_CPU(all, self)); }

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("sum.dim_IntList", TORCH_FN(k_sum_dim));
  m.impl("mean.dim", TORCH_FN(k_mean_dim));
  m.impl("prod.dim_int", TORCH_FN(k_prod_dim));
  m.impl("amax", TORCH_FN(k_amax));
  m.impl("amin", TORCH_FN(k_amin));
  m.impl("max", TORCH_FN(k_max_all));
  m.impl("min", TORCH_FN(k_min_all));
  m.impl("max.dim", TORCH_FN(k_max_dim));
  m.impl("min.dim", TORCH_FN(k_min_dim));
  m.impl("argmax", TORCH_FN(k_argmax));
  m.impl("argmin", TORCH_FN(k_argmin));
  m.impl("norm.ScalarOpt_dim", TORCH_FN(k_norm_dim));
  m.impl("linalg_vector_norm", TORCH_FN(k_linalg_vector_norm));
  m.impl("any", TORCH_FN(k_any));
  m.impl("all", TORCH_FN(k_all));
  m.impl("any.dim", TORCH_FN(k_any_dim));
  m.impl("all.dim", TORCH_FN(k_all_dim));
  m.impl("prod", TORCH_FN(k_prod_all));
  m.impl("norm.ScalarOpt_dim_dtype", TORCH_FN(k_norm_dim_dtype));
}

}  // namespace ops
}  // namespace catch_b200
