// Pooling operators: max_pool2d_with_indices, avg_pool2d, adaptive_avg_pool2d, adaptive_max_pool2d,
// max_pool3d_with_indices, avg_pool3d, adaptive_avg_pool3d (forward and backward).
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

// ---------------------------------------------------------------- 3-D pooling and adaptive max pooling
// One device kernel family (pooling3d.cu) over (N, C, D, H, W); 4-D inputs of the 3-D ops get a batch of one,
// 2-D adaptive max pooling a depth of one.
struct Geo3 {
  int64_t k[3], s[3], p[3], d[3];
};
int64_t pick3(at::IntArrayRef v, int i, int64_t dflt) { return v.empty() ? dflt : (v.size() == 1 ? v[0] : v[i]); }
Geo3 parse3(const char* op, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef p, at::IntArrayRef d) {
  TORCH_CHECK(k.size() == 1 || k.size() == 3, op, ": kernel_size must be a single int, or a tuple of three ints");
  TORCH_CHECK(s.empty() || s.size() == 1 || s.size() == 3, op, ": stride must be omitted, a single int, or a tuple of three ints");
  TORCH_CHECK(p.size() == 1 || p.size() == 3, op, ": padding must be a single int, or a tuple of three ints");
  TORCH_CHECK(d.empty() || d.size() == 1 || d.size() == 3, op, ": dilation must be a single int, or a tuple of three ints");
  Geo3 g;
  for (int i = 0; i < 3; ++i) {
    g.k[i] = pick3(k, i, 1);
    g.s[i] = pick3(s, i, g.k[i]);
    g.p[i] = pick3(p, i, 0);
    g.d[i] = pick3(d, i, 1);
    TORCH_CHECK(g.k[i] > 0 && g.s[i] > 0 && g.d[i] > 0 && g.p[i] >= 0 && g.p[i] * 2 <= g.k[i] * g.d[i] + 1, op,
                ": invalid kernel / stride / padding / dilation");
  }
  return g;
}
Tensor as5d(const Tensor& x) { return x.dim() == 4 ? x.unsqueeze(0) : x; }
bool is_cl3(const Tensor& x) { return x.dim() == 5 && x.stride(1) == 1 && x.size(1) > 1; }
void fill3(B200Pool3Params& p, const Tensor& in5, const Tensor& out5, const Geo3& g) {
  std::memset(&p, 0, sizeof(p));
  p.N = (int)in5.size(0); p.C = (int)in5.size(1);
  for (int i = 0; i < 3; ++i) {
    p.in[i] = (int)in5.size(2 + i); p.out[i] = (int)out5.size(2 + i);
    p.k[i] = (int)g.k[i]; p.s[i] = (int)g.s[i]; p.p[i] = (int)g.p[i]; p.dil[i] = (int)g.d[i];
  }
  for (int i = 0; i < 5; ++i) { p.in_s[i] = in5.stride(i); p.out_s[i] = out5.stride(i); }
  p.channels_last = is_cl3(in5) ? 1 : 0;
  p.dtype = to_b200_dtype(in5.scalar_type());
}
Tensor alloc3(const Tensor& in5, int64_t D, int64_t H, int64_t W, at::ScalarType dt) {
  return empty_b200({in5.size(0), in5.size(1), D, H, W}, dt, in5.device().index(),
                    is_cl3(in5) ? at::MemoryFormat::ChannelsLast3d : at::MemoryFormat::Contiguous);
}
Tensor dense_like(const Tensor& in) {
  return at::empty_strided(in.sizes(), in.is_non_overlapping_and_dense() ? in.strides() : in.contiguous().strides(), in.options());
}
Tensor match_strides(const Tensor& t, const Tensor& like) {
  if (t.strides() == like.strides()) return t;
  return at::empty_strided(like.sizes(), like.strides(), t.options()).copy_(t);
}
void check3(const char* op, const Tensor& self) {
  TORCH_CHECK((self.dim() == 4 || self.dim() == 5) && pool_dtype_ok(self.scalar_type()), "b200 ", op, ": unsupported input ", describe(self));
}

std::tuple<Tensor, Tensor> max_pool3d_device(const Tensor& self, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef pd,
                                             at::IntArrayRef d, bool ceil_mode) {
  check3("max_pool3d", self);
  Geo3 g = parse3("max_pool3d", k, s, pd, d);
  OpScope scope("max_pool3d_with_indices", self);
  Tensor in5 = as5d(self);
  int64_t o[3];
  for (int i = 0; i < 3; ++i) o[i] = at::native::pooling_output_shape<int64_t>(in5.size(2 + i), g.k[i], g.p[i], g.s[i], g.d[i], ceil_mode);
  Tensor out = alloc3(in5, o[0], o[1], o[2], self.scalar_type());
  Tensor idx = alloc3(in5, o[0], o[1], o[2], at::kLong);
  B200Pool3Params p;
  fill3(p, in5, out, g);
  p.is_max = 1;
  B200_KERNEL_CHECK(b200_pool3d_fwd(&p, in5.data_ptr(), out.data_ptr(), i64ptr(idx), scope.stream()));
  if (self.dim() == 4) return {out.squeeze(0), idx.squeeze(0)};
  return {out, idx};
}
std::tuple<Tensor, Tensor> k_max_pool3d_with_indices(const Tensor& self, at::IntArrayRef k, at::IntArrayRef s,
                                                     at::IntArrayRef pd, at::IntArrayRef d, bool ceil_mode) {
  return B200_DISPATCH("max_pool3d_with_indices", max_pool3d_device(self, k, s, pd, d, ceil_mode),
                       B200_CPU(max_pool3d_with_indices, self, k, s, pd, d, ceil_mode));
}
Tensor max_pool3d_bwd_device(const Tensor& grad, const Tensor& self, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef pd,
                             at::IntArrayRef d, const Tensor& indices) {
  check3("max_pool3d_backward", self);
  TORCH_CHECK(grad.scalar_type() == self.scalar_type(), "b200 max_pool3d_backward: dtype mismatch");
  Geo3 g = parse3("max_pool3d", k, s, pd, d);
  OpScope scope("max_pool3d_with_indices_backward", self);
  Tensor in5 = as5d(self), idx5 = as5d(indices);
  Tensor gy = match_strides(as5d(grad), idx5);
  Tensor dx = dense_like(in5);
  B200Pool3Params p;
  fill3(p, dx, idx5, g);
  p.is_max = 1;
  B200_KERNEL_CHECK(b200_pool3d_bwd(&p, gy.data_ptr(), i64ptr(idx5), dx.data_ptr(), scope.stream()));
  return self.dim() == 4 ? dx.squeeze(0) : dx;
}
Tensor k_max_pool3d_with_indices_backward(const Tensor& grad, const Tensor& self, at::IntArrayRef k, at::IntArrayRef s,
                                          at::IntArrayRef pd, at::IntArrayRef d, bool ceil_mode, const Tensor& indices) {
  return B200_DISPATCH("max_pool3d_with_indices_backward", max_pool3d_bwd_device(grad, self, k, s, pd, d, indices),
                       B200_CPU(max_pool3d_with_indices_backward, grad, self, k, s, pd, d, ceil_mode, indices));
}

Tensor avg_pool3d_device(const Tensor& self, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef pd, bool ceil_mode,
                         bool cip, std::optional<int64_t> divisor) {
  check3("avg_pool3d", self);
  Geo3 g = parse3("avg_pool3d", k, s, pd, {});
  OpScope scope("avg_pool3d", self);
  Tensor in5 = as5d(self);
  int64_t o[3];
  for (int i = 0; i < 3; ++i) o[i] = at::native::pooling_output_shape<int64_t>(in5.size(2 + i), g.k[i], g.p[i], g.s[i], 1, ceil_mode);
  Tensor out = alloc3(in5, o[0], o[1], o[2], self.scalar_type());
  B200Pool3Params p;
  fill3(p, in5, out, g);
  p.count_include_pad = cip;
  p.divisor_override = divisor.has_value() ? (int)*divisor : 0;
  B200_KERNEL_CHECK(b200_pool3d_fwd(&p, in5.data_ptr(), out.data_ptr(), nullptr, scope.stream()));
  return self.dim() == 4 ? out.squeeze(0) : out;
}
Tensor k_avg_pool3d(const Tensor& self, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef pd, bool ceil_mode, bool cip,
                    std::optional<int64_t> divisor) {
  return B200_DISPATCH("avg_pool3d", avg_pool3d_device(self, k, s, pd, ceil_mode, cip, divisor),
                       B200_CPU(avg_pool3d, self, k, s, pd, ceil_mode, cip, divisor));
}
Tensor avg_pool3d_bwd_device(const Tensor& grad, const Tensor& self, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef pd,
                             bool cip, std::optional<int64_t> divisor) {
  check3("avg_pool3d_backward", self);
  TORCH_CHECK(grad.scalar_type() == self.scalar_type(), "b200 avg_pool3d_backward: dtype mismatch");
  Geo3 g = parse3("avg_pool3d", k, s, pd, {});
  OpScope scope("avg_pool3d_backward", self);
  Tensor in5 = as5d(self), gy = as5d(grad);
  Tensor dx = dense_like(in5);
  B200Pool3Params p;
  fill3(p, dx, gy, g);
  p.count_include_pad = cip;
  p.divisor_override = divisor.has_value() ? (int)*divisor : 0;
  B200_KERNEL_CHECK(b200_pool3d_bwd(&p, gy.data_ptr(), nullptr, dx.data_ptr(), scope.stream()));
  return self.dim() == 4 ? dx.squeeze(0) : dx;
}
Tensor k_avg_pool3d_backward(const Tensor& grad, const Tensor& self, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef pd,
                             bool ceil_mode, bool cip, std::optional<int64_t> divisor) {
  return B200_DISPATCH("avg_pool3d_backward", avg_pool3d_bwd_device(grad, self, k, s, pd, cip, divisor),
                       B200_CPU(avg_pool3d_backward, grad, self, k, s, pd, ceil_mode, cip, divisor));
}

Tensor adaptive_avg3d_device(const Tensor& self, at::IntArrayRef out_size) {
  check3("adaptive_avg_pool3d", self);
  TORCH_CHECK(out_size.size() == 3, "adaptive_avg_pool3d: output_size must have three elements");
  OpScope scope("_adaptive_avg_pool3d", self);
  Tensor in5 = as5d(self);
  Tensor out = alloc3(in5, out_size[0], out_size[1], out_size[2], self.scalar_type());
  B200Pool3Params p;
  Geo3 g{{1, 1, 1}, {1, 1, 1}, {0, 0, 0}, {1, 1, 1}};
  fill3(p, in5, out, g);
  p.adaptive = 1;
  B200_KERNEL_CHECK(b200_pool3d_fwd(&p, in5.data_ptr(), out.data_ptr(), nullptr, scope.stream()));
  return self.dim() == 4 ? out.squeeze(0) : out;
}
Tensor k_adaptive_avg_pool3d(const Tensor& self, c10::SymIntArrayRef out_size) {
  auto sz = C10_AS_INTARRAYREF_SLOW(out_size);
  return B200_DISPATCH("_adaptive_avg_pool3d", adaptive_avg3d_device(self, sz), B200_CPU_SYMINT(_adaptive_avg_pool3d, self, out_size));
}
Tensor adaptive_avg3d_bwd_device(const Tensor& grad, const Tensor& self) {
  check3("adaptive_avg_pool3d_backward", self);
  TORCH_CHECK(grad.scalar_type() == self.scalar_type(), "b200 adaptive_avg_pool3d_backward: dtype mismatch");
  OpScope scope("_adaptive_avg_pool3d_backward", self);
  Tensor in5 = as5d(self), gy = as5d(grad);
  Tensor dx = dense_like(in5);
  B200Pool3Params p;
  Geo3 g{{1, 1, 1}, {1, 1, 1}, {0, 0, 0}, {1, 1, 1}};
  fill3(p, dx, gy, g);
  p.adaptive = 1;
  B200_KERNEL_CHECK(b200_pool3d_bwd(&p, gy.data_ptr(), nullptr, dx.data_ptr(), scope.stream()));
  return self.dim() == 4 ? dx.squeeze(0) : dx;
}
Tensor k_adaptive_avg_pool3d_backward(const Tensor& grad, const Tensor& self) {
  return B200_DISPATCH("_adaptive_avg_pool3d_backward", adaptive_avg3d_bwd_device(grad, self),
                       B200_CPU(_adaptive_avg_pool3d_backward, grad, self));
}

// 2-D adaptive max pooling: the 3-D kernel with a depth of one
std::tuple<Tensor, Tensor> adaptive_max2d_device(const Tensor& self, at::IntArrayRef out_size) {
  TORCH_CHECK((self.dim() == 3 || self.dim() == 4) && pool_dtype_ok(self.scalar_type()) && out_size.size() == 2,
              "b200 adaptive_max_pool2d: unsupported input ", describe(self));
  OpScope scope("adaptive_max_pool2d", self);
  Tensor in4 = as4d(self);
  Tensor out = alloc_like_layout(in4, out_size[0], out_size[1], self.scalar_type());
  Tensor idx = alloc_like_layout(in4, out_size[0], out_size[1], at::kLong);
  Tensor in5 = in4.unsqueeze(2), out5 = out.unsqueeze(2);
  B200Pool3Params p;
  Geo3 g{{1, 1, 1}, {1, 1, 1}, {0, 0, 0}, {1, 1, 1}};
  fill3(p, in5, out5, g);
  p.channels_last = is_cl(in4) ? 1 : 0;
  p.adaptive = 1;
  p.is_max = 1;
  B200_KERNEL_CHECK(b200_pool3d_fwd(&p, in4.data_ptr(), out.data_ptr(), i64ptr(idx), scope.stream()));
  if (self.dim() == 3) return {out.squeeze(0), idx.squeeze(0)};
  return {out, idx};
}
std::tuple<Tensor, Tensor> k_adaptive_max_pool2d(const Tensor& self, at::IntArrayRef out_size) {
  return B200_DISPATCH("adaptive_max_pool2d", adaptive_max2d_device(self, out_size), B200_CPU(adaptive_max_pool2d, self, out_size));
}
Tensor adaptive_max2d_bwd_device(const Tensor& grad, const Tensor& self, const Tensor& indices) {
  TORCH_CHECK(pool_dtype_ok(self.scalar_type()) && grad.scalar_type() == self.scalar_type(), "b200 adaptive_max_pool2d_backward: unsupported dtype");
  OpScope scope("adaptive_max_pool2d_backward", self);
  Tensor in4 = as4d(self), idx4 = as4d(indices);
  Tensor gy = match_strides(as4d(grad), idx4);
  Tensor dx = dense_like(in4);
  B200Pool3Params p;
  Geo3 g{{1, 1, 1}, {1, 1, 1}, {0, 0, 0}, {1, 1, 1}};
  fill3(p, dx.unsqueeze(2), idx4.unsqueeze(2), g);
  p.channels_last = is_cl(dx) ? 1 : 0;
  p.adaptive = 1;
  p.is_max = 1;
  B200_KERNEL_CHECK(b200_pool3d_bwd(&p, gy.data_ptr(), i64ptr(idx4), dx.data_ptr(), scope.stream()));
  return self.dim() == 3 ? dx.squeeze(0) : dx;
}
Tensor k_adaptive_max_pool2d_backward(const Tensor& grad, const Tensor& self, const Tensor& indices) {
  return B200_DISPATCH("adaptive_max_pool2d_backward", adaptive_max2d_bwd_device(grad, self, indices),
                       B200_CPU(adaptive_max_pool2d_backward, grad, self, indices));
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
  m.impl("max_pool3d_with_indices", TORCH_FN(k_max_pool3d_with_indices));
  m.impl("max_pool3d_with_indices_backward", TORCH_FN(k_max_pool3d_with_indices_backward));
  m.impl("avg_pool3d", TORCH_FN(k_avg_pool3d));
  m.impl("avg_pool3d_backward", TORCH_FN(k_avg_pool3d_backward));
  m.impl("_adaptive_avg_pool3d", TORCH_FN(k_adaptive_avg_pool3d));
  m.impl("_adaptive_avg_pool3d_backward", TORCH_FN(k_adaptive_avg_pool3d_backward));
  m.impl("adaptive_max_pool2d", TORCH_FN(k_adaptive_max_pool2d));
  m.impl("adaptive_max_pool2d_backward", TORCH_FN(k_adaptive_max_pool2d_backward));
}

}  // namespace ops
}  // namespace catch_b200
