// Pooling operators: max_pool2d_with_indices, avg_pool2d, adaptive_avg_pool2d
// (forward and backward).
//
// Parity: torch_mlu/csrc/aten/operators/cnnl/pooling.cpp:48-290 and
// adaptive_pooling.cpp.  Indices are flattened h*W+w positions and ceil_mode clamps
// windows, unlike the reference's window-local indices and padding emulation.
#include <ATen/native/Pool.h>
#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

bool pool_dtype_ok(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf; }

struct Geo {
  int64_t kh, kw, sh, sw, ph, pw, dh, dw;
};
Geo parse(at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef p, at::IntArrayRef d) {
  Geo g;
  TORCH_CHECK(k.size() == 1 || k.size() == 2, "pool2d: kernel_size must either be a single int, or a tuple of two ints");
  g.kh = k[0]; g.kw = k.size() == 1 ? k[0] : k[1];
  TORCH_CHECK(s.empty() || s.size() == 1 || s.size() == 2, "pool2d: stride must either be omitted, a single int, or a tuple of two ints");
  g.sh = s.empty() ? g.kh : s[0]; g.sw = s.empty() ? g.kw : (s.size() == 1 ? s[0] : s[1]);
  TORCH_CHECK(p.size() == 1 || p.size() == 2, "pool2d: padding must either be a single int, or a tuple of two ints");
  g.ph = p[0]; g.pw = p.size() == 1 ? p[0] : p[1];
  g.dh = d.empty() ? 1 : d[0]; g.dw = d.empty() ? 1 : (d.size() == 1 ? d[0] : d[1]);
  return g;
}

// 4-D view (a 3-D input gets a leading batch of 1)
Tensor as4d(const Tensor& x) { return x.dim() == 3 ? x.unsqueeze(0) : x; }
bool is_cl(const Tensor& x) { return x.dim() == 4 && x.stride(1) == 1 && x.size(1) > 1; }

void fill(B200PoolParams& p, const Tensor& in4, const Tensor& out4, const Geo& g) {
  std::memset(&p, 0, sizeof(p));
  p.N = (int)in4.size(0); p.C = (int)in4.size(1); p.H = (int)in4.size(2); p.W = (int)in4.size(3);
  p.P = (int)out4.size(2); p.Q = (int)out4.size(3);
  p.kh = (int)g.kh; p.kw = (int)g.kw; p.sh = (int)g.sh; p.sw = (int)g.sw; p.ph = (int)g.ph; p.pw = (int)g.pw;
  p.dh = (int)g.dh; p.dw = (int)g.dw;
  for (int i = 0; i < 4; ++i) { p.in_s[i] = in4.stride(i); p.out_s[i] = out4.stride(i); }
  p.channels_last = is_cl(in4) ? 1 : 0;
  p.dtype = to_b200_dtype(in4.scalar_type());
}

Tensor alloc_like_layout(const Tensor& in4, int64_t P, int64_t Q, at::ScalarType dt) {
  return empty_b200({in4.size(0), in4.size(1), P, Q}, dt, in4.device().index(),
                    is_cl(in4) ? at::MemoryFormat::ChannelsLast : at::MemoryFormat::Contiguous);
}

std::tuple<Tensor, Tensor> max_pool_device(const Tensor& self, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef pd,
                                           at::IntArrayRef d, bool ceil_mode) {
  TORCH_CHECK((self.dim() == 3 || self.dim() == 4) && pool_dtype_ok(self.scalar_type()), "b200 max_pool2d: unsupported input ", describe(self));
  Geo g = parse(k, s, pd, d);
  OpScope scope("max_pool2d_with_indices", self);
  Tensor in4 = as4d(self);
  const int64_t P = at::native::pooling_output_shape<int64_t>(in4.size(2), g.kh, g.ph, g.sh, g.dh, ceil_mode);
  const int64_t Q = at::native::pooling_output_shape<int64_t>(in4.size(3), g.kw, g.pw, g.sw, g.dw, ceil_mode);
  Tensor out = alloc_like_layout(in4, P, Q, self.scalar_type());
  Tensor idx = alloc_like_layout(in4, P, Q, at::kLong);
  B200PoolParams p;
  fill(p, in4, out, g);
  B200_KERNEL_CHECK(b200_maxpool2d_fwd(&p, in4.data_ptr(), out.data_ptr(), i64ptr(idx), scope.stream()));
  if (self.dim() == 3) return {out.squeeze(0), idx.squeeze(0)};
  return {out, idx};
}
std::tuple<Tensor, Tensor> k_max_pool2d_with_indices(const Tensor& self, at::IntArrayRef k, at::IntArrayRef s,
                                                     at::IntArrayRef pd, at::IntArrayRef d, bool ceil_mode) {
  return B200_DISPATCH("max_pool2d_with_indices", max_pool_device(self, k, s, pd, d, ceil_mode),
                       B200_CPU(max_pool2d_with_indices, self, k, s, pd, d, ceil_mode));
}

Tensor max_pool_bwd_device(const Tensor& grad, const Tensor& self, at::IntArrayRef k, at::IntArrayRef s,
                           at::IntArrayRef pd, at::IntArrayRef d, bool, const Tensor& indices) {
  TORCH_CHECK(pool_dtype_ok(self.scalar_type()) && grad.scalar_type() == self.scalar_type(), "b200 max_pool2d_backward: unsupported dtype");
  Geo g = parse(k, s, pd, d);
  OpScope scope("max_pool2d_with_indices_backward", self);
  Tensor in4 = as4d(self), idx4 = as4d(indices);
  Tensor gy = as4d(grad);
  if (gy.strides() != idx4.strides()) gy = at::empty_strided(idx4.sizes(), idx4.strides(), grad.options()).copy_(gy);
  Tensor dx = at::empty_strided(in4.sizes(), in4.is_non_overlapping_and_dense() ? in4.strides() : in4.contiguous().strides(), self.options());
  B200PoolParams p;
  fill(p, dx, idx4, g);
  B200_KERNEL_CHECK(b200_maxpool2d_bwd(&p, gy.data_ptr(), i64ptr(idx4), dx.data_ptr(), scope.stream()));
  return self.dim() == 3 ? dx.squeeze(0) : dx;
}
Tensor k_max_pool2d_with_indices_backward(const Tensor& grad, const Tensor& self, at::IntArrayRef k, at::IntArrayRef s,
                                          at::IntArrayRef pd, at::IntArrayRef d, bool ceil_mode, const Tensor& indices) {
  return B200_DISPATCH("max_pool2d_with_indices_backward", max_pool_bwd_device(grad, self, k, s, pd, d, ceil_mode, indices),
                       B200_CPU(max_pool2d_with_indices_backward, grad, self, k, s, pd, d, ceil_mode, indices));
}

Tensor avg_pool_device(const Tensor& self, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef pd, bool ceil_mode,
                       bool count_include_pad, std::optional<int64_t> divisor) {
  TORCH_CHECK((self.dim() == 3 || self.dim() == 4) && pool_dtype_ok(self.scalar_type()), "b200 avg_pool2d: unsupported input ", describe(self));
  Geo g = parse(k, s, pd, {});
  OpScope scope("avg_pool2d", self);
  Tensor in4 = as4d(self);
  const int64_t P = at::native::pooling_output_shape<int64_t>(in4.size(2), g.kh, g.ph, g.sh, 1, ceil_mode);
  const int64_t Q = at::native::pooling_output_shape<int64_t>(in4.size(3), g.kw, g.pw, g.sw, 1, ceil_mode);
  Tensor out = alloc_like_layout(in4, P, Q, self.scalar_type());
  B200PoolParams p;
  fill(p, in4, out, g);
  p.count_include_pad = count_include_pad;
  p.divisor_override = divisor.has_value() ? (int)*divisor : 0;
  B200_KERNEL_CHECK(b200_avgpool2d_fwd(&p, in4.data_ptr(), out.data_ptr(), scope.stream()));
  return self.dim() == 3 ? out.squeeze(0) : out;
}
Tensor k_avg_pool2d(const Tensor& self, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef pd, bool ceil_mode,
                    bool cip, std::optional<int64_t> divisor) {
  return B200_DISPATCH("avg_pool2d", avg_pool_device(self, k, s, pd, ceil_mode, cip, divisor),
                       B200_CPU(avg_pool2d, self, k, s, pd, ceil_mode, cip, divisor));
}
Tensor avg_pool_bwd_device(const Tensor& grad, const Tensor& self, at::IntArrayRef k, at::IntArrayRef s,
                           at::IntArrayRef pd, bool, bool cip, std::optional<int64_t> divisor) {
  TORCH_CHECK(pool_dtype_ok(self.scalar_type()) && grad.scalar_type() == self.scalar_type(), "b200 avg_pool2d_backward: unsupported dtype");
  Geo g = parse(k, s, pd, {});
  OpScope scope("avg_pool2d_backward", self);
  Tensor in4 = as4d(self), gy = as4d(grad);
  Tensor dx = at::empty_strided(in4.sizes(), in4.is_non_overlapping_and_dense() ? in4.strides() : in4.contiguous().strides(), self.options());
  B200PoolParams p;
  fill(p, dx, gy, g);
  p.count_include_pad = cip;
  p.divisor_override = divisor.has_value() ? (int)*divisor : 0;
  B200_KERNEL_CHECK(b200_avgpool2d_bwd(&p, gy.data_ptr(), dx.data_ptr(), scope.stream()));
  return self.dim() == 3 ? dx.squeeze(0) : dx;
}
Tensor k_avg_pool2d_backward(const Tensor& grad, const Tensor& self, at::IntArrayRef k, at::IntArrayRef s,
                             at::IntArrayRef pd, bool ceil_mode, bool cip, std::optional<int64_t> divisor) {
  return B200_DISPATCH("avg_pool2d_backward", avg_pool_bwd_device(grad, self, k, s, pd, ceil_mode, cip, divisor),
                       B200_CPU(avg_pool2d_backward, grad, self, k, s, pd, ceil_mode, cip, divisor));
}

Tensor adaptive_device(const Tensor& self, at::IntArrayRef out_size) {
  TORCH_CHECK((self.dim() == 3 || self.dim() == 4) && pool_dtype_ok(self.scalar_type()) && out_size.size() == 2,
              "b200 adaptive_avg_pool2d: unsupported input ", describe(self));
  OpScope scope("_adaptive_avg_pool2d", self);
  Tensor in4 = as4d(self);
  Tensor out = alloc_like_layout(in4, out_size[0], out_size[1], self.scalar_type());
  B200PoolParams p;
  Geo g{1, 1, 1, 1, 0, 0, 1, 1};
  fill(p, in4, out, g);
  B200_KERNEL_CHECK(b200_adaptive_avgpool2d_fwd(&p, in4.data_ptr(), out.data_ptr(), scope.stream()));
  return self.dim() == 3 ? out.squeeze(0) : out;
}
Tensor k_adaptive_avg_pool2d(const Tensor& self, c10::SymIntArrayRef out_size) {
  auto sz = C10_AS_INTARRAYREF_SLOW(out_size);
  return B200_DISPATCH("_adaptive_avg_pool2d", adaptive_device(self, sz), B200_CPU_SYMINT(_adaptive_avg_pool2d, self, out_size));
}
Tensor adaptive_bwd_device(const Tensor& grad, const Tensor& self) {
  TORCH_CHECK(pool_dtype_ok(self.scalar_type()) && grad.scalar_type() == self.scalar_type(), "b200 adaptive_avg_pool2d_backward: unsupported dtype");
  OpScope scope("_adaptive_avg_pool2d_backward", self);
  Tensor in4 = as4d(self), gy = as4d(grad);
  Tensor dx = at::empty_strided(in4.sizes(), in4.is_non_overlapping_and_dense() ? in4.strides() : in4.contiguous().strides(), self.options());
  B200PoolParams p;
  Geo g{1, 1, 1, 1, 0, 0, 1, 1};
  fill(p, dx, gy, g);
  B200_KERNEL_CHECK(b200_adaptive_avgpool2d_bwd(&p, gy.data_ptr(), dx.data_ptr(), scope.stream()));
  return self.dim() == 3 ? dx.squeeze(0) : dx;
}
Tensor k_adaptive_avg_pool2d_backward(const Tensor& grad, const Tensor& self) {
  return B200_DISPATCH("_adaptive_avg_pool2d_backward", adaptive_bwd_device(grad, self),
                       B200_CPU(_adaptive_avg_pool2d_backward, grad, self));
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("max_pool2d_with_indices", TORCH_FN(k_max_pool2d_with_indices));
  m.impl("max_pool2d_with_indices_backward", TORCH_FN(k_max_pool2d_with_indices_backward));
  m.impl("avg_pool2d", TORCH_FN(k_avg_pool2d));
  m.impl("avg_pool2d_backward", TORCH_FN(k_avg_pool2d_backward));
  m.impl("_adaptive_avg_pool2d", TORCH_FN(k_adaptive_avg_pool2d));
  m.impl("_adaptive_avg_pool2d_backward", TORCH_FN(k_adaptive_avg_pool2d_backward));
}

}  // namespace ops
}  // namespace catch_b200
