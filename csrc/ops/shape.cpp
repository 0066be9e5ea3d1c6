// Data-movement operators built on the strided copy kernel: cat (stack / hstack /
// vstack decompose to it), repeat and constant padding stay composite.
// Parity: torch_mlu/csrc/aten/operators/cnnl/cat.cpp:60 (cnnlConcat).
#include <ATen/WrapDimUtils.h>
#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

Tensor cat_device(const at::ITensorListRef& tensors, int64_t dim) {
  std::vector<Tensor> ts;
  for (const Tensor& t : tensors) ts.push_back(t);
  TORCH_CHECK(!ts.empty(), "torch.cat(): expected a non-empty list of Tensors");
  // legacy rule: 1-D empty tensors are skipped
  std::vector<Tensor> valid;
  at::ScalarType dt = ts[0].scalar_type();
  for (auto& t : ts) {
    dt = at::promote_types(dt, t.scalar_type());
    if (!(t.dim() == 1 && t.numel() == 0)) valid.push_back(t);
  }
  if (valid.empty()) return empty_b200({0}, dt, ts[0].device().index());
  const int64_t nd = valid[0].dim();
  dim = at::maybe_wrap_dim(dim, nd);
  std::vector<int64_t> shape(valid[0].sizes().begin(), valid[0].sizes().end());
  int64_t total = 0;
  for (auto& t : valid) {
    TORCH_CHECK(t.dim() == nd, "Tensors must have same number of dimensions: got ", nd, " and ", t.dim());
    for (int64_t d = 0; d < nd; ++d)
      TORCH_CHECK(d == dim || t.size(d) == shape[d], "Sizes of tensors must match except in dimension ", dim);
    TORCH_CHECK(is_b200(t) && t.device() == valid[0].device(), "cat: all tensors must be on the same blackwell device");
    total += t.size(dim);
  }
  shape[dim] = total;
  OpScope scope("cat", valid[0]);
  const bool cl = nd == 4 && valid[0].is_contiguous(at::MemoryFormat::ChannelsLast) && !valid[0].is_contiguous();
  Tensor out = empty_b200(shape, dt, valid[0].device().index(), cl ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous);
  int64_t off = 0;
  for (auto& t : valid) {
    if (t.size(dim) == 0) continue;
    Tensor dst = out.narrow(dim, off, t.size(dim));
    if (dst.numel()) launch_copy(t, dst, scope.stream());
    off += t.size(dim);
  }
  return out;
}
Tensor k_cat(const at::ITensorListRef& tensors, int64_t dim) {
  return B200_DISPATCH("cat", cat_device(tensors, dim), B200_CPU(cat, tensors, dim));
}
Tensor& k_cat_out(const at::ITensorListRef& tensors, int64_t dim, Tensor& out) {
  Tensor r = k_cat(tensors, dim);
  out.resize_(r.sizes());
  out.copy_(r);
  return out;
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("cat", TORCH_FN(k_cat));
  m.impl("cat.out", TORCH_FN(k_cat_out));
}

}  // namespace ops
}  // namespace catch_b200
