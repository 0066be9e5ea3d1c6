// gather / scatter, advanced indexing (index, index_put), nonzero, masked_select, arange,
// tril / triu, sort / topk, nearest and bilinear 2-D resampling, NMS.
//
// Parity: torch_mlu/csrc/aten/operators/cnnl/{index.cpp,index_put.cpp,masked_select.cpp,
// nonzero.cpp,arange.cpp,tril.cpp,triu.cpp,topk.cpp,sort.cpp,upsample_nearest2d.cpp,
// upsample_bilinear2d.cpp,nms.cpp}.  Cases the device kernels do not cover (indexed
// dimensions that are not adjacent, rows longer than the sort kernel's limit, integer
// accumulation) raise and are rerun on the CPU by the per-op fallback.
#include <ATen/ExpandUtils.h>
#include <ATen/core/op_registration/op_registration.h>
#include <torch/library.h>

#include "../runtime/caching_allocator.h"
#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

bool float_type(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf; }

// One int32 flag per device that the kernels set when they meet an index out of range (the access
// is skipped).  It is read, reported and cleared when the backend runs in synchronous mode.
std::mutex g_flag_mu;
std::vector<Tensor> g_flags(64);
const bool g_flag_dropper = [] {
  registerCacheDropper([] {  // torch.blackwell.empty_cache() releases the flags; they are recreated on demand
    std::lock_guard<std::mutex> lk(g_flag_mu);
    for (auto& f : g_flags) f = Tensor();
  });
  return true;
}();
Tensor bad_index_flag(int device) {
  std::lock_guard<std::mutex> lk(g_flag_mu);
  Tensor& f = g_flags[device & 63];
  if (!f.defined()) f = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(c10::Device(c10::DeviceType::PrivateUse1, device)));
  return f;
}
void check_bad_index(const char* op, int device) {
  if (!flags().async_disable) return;
  Tensor f = bad_index_flag(device);
  if (f.item<int>() != 0) {
    f.zero_();
    TORCH_CHECK_INDEX(false, op, ": index out of range");
  }
}
int* bad_ptr(const Tensor& like) { return bad_index_flag(like.device().index()).data_ptr<int>(); }

std::vector<long long> ll(at::IntArrayRef v) { return std::vector<long long>(v.begin(), v.end()); }

// ---- gather / scatter ----------------------------------------------------------------
void run_dim_index(const Tensor& a, const Tensor& b, const Tensor& index, int64_t dim, int mode, const OpScope& scope) {
  auto sizes = ll(index.sizes()), as = ll(a.strides()), bs = ll(b.strides());
  B200_KERNEL_CHECK(b200_dim_index(a.data_ptr(), b.data_ptr(), (int)a.element_size(), i64ptr(index), (int)index.dim(), (int)dim,
                                   sizes.data(), as.data(), bs.data(), a.size(dim), mode, bad_ptr(a), scope.stream()));
}

Tensor gather_device(const Tensor& self_in, int64_t dim, const Tensor& index_in) {
  TORCH_CHECK(index_in.scalar_type() == at::kLong, "gather: index must be int64");
  Tensor self = self_in.dim() == 0 ? self_in.unsqueeze(0) : self_in;
  Tensor index = (index_in.dim() == 0 ? index_in.unsqueeze(0) : index_in).contiguous();
  TORCH_CHECK(self.dim() == index.dim() && self.dim() <= 8, "gather: index and input must have the same rank (<= 8)");
  dim = at::maybe_wrap_dim(dim, self.dim());
  OpScope scope("gather", self);
  Tensor out = empty_b200(index.sizes(), self.scalar_type(), self.device().index());
  if (index.numel() > 0) run_dim_index(self, out, index, dim, 0, scope);
  check_bad_index("gather", self.device().index());
  return index_in.dim() == 0 ? out.squeeze(0) : out;
}
Tensor k_gather(const Tensor& self, int64_t dim, const Tensor& index, bool sparse_grad) {
  check_same_device("gather", self, index);
  return B200_DISPATCH("gather", gather_device(self, dim, index), B200_CPU(gather, self, dim, index, sparse_grad));
}

Tensor& scatter_device_(Tensor& self, int64_t dim, const Tensor& index_in, const Tensor& src, bool add) {
  TORCH_CHECK(index_in.scalar_type() == at::kLong, "scatter: index must be int64");
  TORCH_CHECK(self.dim() == index_in.dim() && src.dim() == index_in.dim() && self.dim() >= 1 && self.dim() <= 8,
              "scatter: input, index and src must have the same rank (1..8)");
  TORCH_CHECK(src.scalar_type() == self.scalar_type(), "scatter: src and self must have the same dtype");
  dim = at::maybe_wrap_dim(dim, self.dim());
  OpScope scope(add ? "scatter_add" : "scatter", self);
  Tensor index = index_in.contiguous();
  if (index.numel() == 0) return self;
  if (!add) {
    run_dim_index(self, src, index, dim, 1, scope);
  } else if (self.scalar_type() == at::kFloat) {
    run_dim_index(self, src, index, dim, 2, scope);
  } else {
    TORCH_CHECK(float_type(self.scalar_type()), "scatter_add: integer accumulation has no device kernel");
    Tensor acc = self.to(at::kFloat), s32 = src.to(at::kFloat);
    run_dim_index(acc, s32, index, dim, 2, scope);
    self.copy_(acc);
  }
  check_bad_index("scatter", self.device().index());
  return self;
}
Tensor& k_scatter_src_(Tensor& self, int64_t dim, const Tensor& index, const Tensor& src) {
  check_same_device("scatter", self, index, src);
  B200_DISPATCH("scatter_.src", (void)scatter_device_(self, dim, index, src, false), (void)B200_CPU(scatter__src, self, dim, index, src));
  return self;
}
Tensor k_scatter_src(const Tensor& self, int64_t dim, const Tensor& index, const Tensor& src) {
  Tensor out = self.clone();
  return k_scatter_src_(out, dim, index, src);
}
Tensor& k_scatter_value_(Tensor& self, int64_t dim, const Tensor& index, const at::Scalar& value) {
  check_same_device("scatter", self, index);
  B200_DISPATCH("scatter_.value", (void)scatter_device_(self, dim, index, at::full(index.sizes(), value, self.options()), false),
                (void)B200_CPU(scatter__value, self, dim, index, value));
  return self;
}
Tensor k_scatter_value(const Tensor& self, int64_t dim, const Tensor& index, const at::Scalar& value) {
  Tensor out = self.clone();
  return k_scatter_value_(out, dim, index, value);
}
Tensor& k_scatter_add_(Tensor& self, int64_t dim, const Tensor& index, const Tensor& src) {
  check_same_device("scatter_add", self, index, src);
  B200_DISPATCH("scatter_add_", (void)scatter_device_(self, dim, index, src, true), (void)B200_CPU(scatter_add_, self, dim, index, src));
  return self;
}
Tensor k_scatter_add(const Tensor& self, int64_t dim, const Tensor& index, const Tensor& src) {
  Tensor out = self.clone();
  return k_scatter_add_(out, dim, index, src);
}

// ---- nonzero / masked_select ----------------------------------------------------------
Tensor nonzero_device(const Tensor& self) {
  OpScope scope("nonzero", self);
  TORCH_CHECK(self.dim() <= 8 && !self.is_complex(), "nonzero: unsupported input");
  Tensor x = self.contiguous();
  const int64_t n = x.numel();
  const int ndim = (int)x.dim();
  auto lopt = self.options().dtype(at::kLong);
  if (n == 0) return at::empty({0, ndim}, lopt);
  Tensor ws = at::empty({(int64_t)b200_nonzero_workspace_elems(n)}, lopt);
  const int is_float = at::isFloatingType(x.scalar_type()) ? 1 : 0;
  B200_KERNEL_CHECK(b200_nonzero_count(x.data_ptr(), (int)x.element_size(), is_float, n, i64ptr(ws), scope.stream()));
  const int64_t total = ws[ws.numel() - 1].item<int64_t>();  // the output size is data dependent: one synchronisation
  Tensor out = at::empty({total, ndim}, lopt);
  if (total > 0 && ndim > 0) {
    auto sizes = ll(x.sizes());
    B200_KERNEL_CHECK(b200_nonzero_write(x.data_ptr(), (int)x.element_size(), is_float, n, i64ptr(ws), ndim, sizes.data(),
                                         i64ptr(out), scope.stream()));
  }
  return out;
}
Tensor k_nonzero(const Tensor& self) { return B200_DISPATCH("nonzero", nonzero_device(self), B200_CPU(nonzero, self)); }

Tensor take_flat(const Tensor& src_flat, const Tensor& idx, const OpScope& scope) {
  Tensor out = empty_b200({idx.numel()}, src_flat.scalar_type(), src_flat.device().index());
  B200_KERNEL_CHECK(b200_take_rows(src_flat.data_ptr(), i64ptr(idx), 1, src_flat.numel(), idx.numel(),
                                   (long long)src_flat.element_size(), out.data_ptr(), bad_ptr(src_flat), scope.stream()));
  return out;
}
Tensor masked_select_device(const Tensor& self, const Tensor& mask) {
  TORCH_CHECK(mask.scalar_type() == at::kBool, "masked_select: mask must be a bool tensor");
  auto [m, s] = at::expand_outplace(mask, self);
  Tensor idx = nonzero_device(m->contiguous().view({-1})).view({-1});
  OpScope scope("masked_select", self);
  return take_flat(s->contiguous().view({-1}), idx, scope);
}
Tensor k_masked_select(const Tensor& self, const Tensor& mask) {
  check_same_device("masked_select", self, mask);
  return B200_DISPATCH("masked_select", masked_select_device(self, mask), B200_CPU(masked_select, self, mask));
}

// ---- advanced indexing ------------------------------------------------------------------
struct LinearIndex {
  Tensor linear;                 // int64, broadcast shape of the index tensors, values in [0, n_indexed)
  int64_t first = 0, count = 0;  // indexed dimensions [first, first + count)
  int64_t outer = 1, n_indexed = 1, inner = 1;
  std::vector<int64_t> result_shape;
};
// Index tensors on adjacent dimensions are folded into one linear index over those dimensions.
LinearIndex linearize(const Tensor& self, const c10::List<std::optional<Tensor>>& indices) {
  std::vector<Tensor> per_dim;  // undefined = slice
  for (size_t i = 0; i < indices.size(); ++i) {
    std::optional<Tensor> oi = indices.get(i);
    if (!oi.has_value() || !oi->defined()) { per_dim.emplace_back(); continue; }
    const Tensor& t = *oi;
    if (t.scalar_type() == at::kBool || t.scalar_type() == at::kByte) {
      // a mask over k dimensions is k index tensors
      for (int64_t d = 0; d < t.dim(); ++d)
        TORCH_CHECK_INDEX(t.size(d) == self.size((int64_t)per_dim.size() + d), "index: mask shape does not match the indexed tensor");
      Tensor m = t.device() == self.device() ? t : t.to(self.device());  // a mask on the host is accepted, like an index
      Tensor nz = nonzero_device(m.scalar_type() == at::kBool ? m : m.ne(0));
      for (int64_t d = 0; d < t.dim(); ++d) per_dim.push_back(nz.select(1, d));
    } else {
      TORCH_CHECK(t.scalar_type() == at::kLong || t.scalar_type() == at::kInt, "index: tensors used as indices must be long, int, byte or bool");
      per_dim.push_back(t.scalar_type() == at::kLong ? t : t.to(at::kLong));
    }
  }
  TORCH_CHECK_INDEX((int64_t)per_dim.size() <= self.dim(), "too many indices for tensor of dimension ", self.dim());
  while ((int64_t)per_dim.size() < self.dim()) per_dim.emplace_back();
  LinearIndex r;
  int64_t first = -1, last = -1;
  for (int64_t d = 0; d < self.dim(); ++d)
    if (per_dim[d].defined()) { if (first < 0) first = d; last = d; }
  TORCH_CHECK(first >= 0, "index: no index tensor given");
  for (int64_t d = first; d <= last; ++d)
    TORCH_CHECK(per_dim[d].defined(), "b200 index: indexed dimensions must be adjacent for the device kernel");
  r.first = first; r.count = last - first + 1;
  std::vector<Tensor> idx(per_dim.begin() + first, per_dim.begin() + last + 1);
  for (auto& t : idx) t = t.to(self.device());
  std::vector<Tensor> b = at::expand_outplace(idx);
  Tensor lin;
  int64_t stride = 1;
  for (int64_t k = r.count - 1; k >= 0; --k) {
    const int64_t size = self.size(first + k);
    Tensor t = at::where(b[k].lt(0), b[k].add(size), b[k]);
    lin = lin.defined() ? lin.add(t, stride) : (stride == 1 ? t : t.mul(stride));
    stride *= size;
  }
  r.linear = lin.contiguous();
  r.n_indexed = stride;
  for (int64_t d = 0; d < first; ++d) { r.outer *= self.size(d); r.result_shape.push_back(self.size(d)); }
  for (auto s : r.linear.sizes()) r.result_shape.push_back(s);
  for (int64_t d = last + 1; d < self.dim(); ++d) { r.inner *= self.size(d); r.result_shape.push_back(self.size(d)); }
  return r;
}

Tensor index_device(const Tensor& self, const c10::List<std::optional<Tensor>>& indices) {
  LinearIndex li = linearize(self, indices);
  OpScope scope("index", self);
  Tensor src = self.contiguous();
  Tensor out = empty_b200(li.result_shape, self.scalar_type(), self.device().index());
  if (out.numel() > 0) {
    B200_KERNEL_CHECK(b200_take_rows(src.data_ptr(), i64ptr(li.linear), li.outer, li.n_indexed, li.linear.numel(),
                                     li.inner * (long long)src.element_size(), out.data_ptr(), bad_ptr(self), scope.stream()));
  }
  check_bad_index("index", self.device().index());
  return out;
}
Tensor k_index(const Tensor& self, const c10::List<std::optional<Tensor>>& indices) {
  return B200_DISPATCH("index.Tensor", index_device(self, indices), B200_CPU(index_Tensor, self, indices));
}

Tensor& index_put_device_(Tensor& self, const c10::List<std::optional<Tensor>>& indices, const Tensor& values, bool accumulate) {
  LinearIndex li = linearize(self, indices);
  OpScope scope("index_put", self);
  if (li.linear.numel() == 0 || self.numel() == 0) return self;
  Tensor vals = values.to(self.device(), self.scalar_type()).expand(li.result_shape).contiguous();
  const bool acc16 = accumulate && self.scalar_type() != at::kFloat;
  if (acc16) TORCH_CHECK(float_type(self.scalar_type()), "index_put(accumulate=True): integer accumulation has no device kernel");
  Tensor dst = acc16 ? self.to(at::kFloat).contiguous() : (self.is_contiguous() ? self : self.contiguous());
  if (acc16) vals = vals.to(at::kFloat);
  B200_KERNEL_CHECK(b200_put_rows(dst.data_ptr(), i64ptr(li.linear), li.outer, li.n_indexed, li.linear.numel(), li.inner,
                                  (int)dst.element_size(), vals.data_ptr(), accumulate ? 1 : 0, bad_ptr(self), scope.stream()));
  if (!dst.is_same(self)) self.copy_(dst);
  check_bad_index("index_put", self.device().index());
  return self;
}
Tensor& k_index_put_impl_(Tensor& self, const c10::List<std::optional<Tensor>>& indices, const Tensor& values, bool accumulate,
                          bool unsafe) {
  B200_DISPATCH("_index_put_impl_", (void)index_put_device_(self, indices, values, accumulate),
                (void)B200_CPU(_index_put_impl_, self, indices, values, accumulate, unsafe));
  return self;
}

// ---- arange, tril / triu ------------------------------------------------------------------
Tensor& arange_out_device(const at::Scalar& start, const at::Scalar& end, const at::Scalar& step, Tensor& out) {
  const double s = start.toDouble(), e = end.toDouble(), st = step.toDouble();
  TORCH_CHECK(st != 0 && ((st > 0 && e >= s) || (st < 0 && e <= s)), "arange: upper bound and larger bound inconsistent with step sign");
  const int64_t n = (int64_t)std::ceil((e - s) / st);
  const auto t = out.scalar_type();
  TORCH_CHECK(float_type(t) || t == at::kDouble || t == at::kLong || t == at::kInt, "arange: unsupported dtype ", t);
  if (out.numel() != n) out.resize_({n});
  OpScope scope("arange", out);
  Tensor dst = out.is_contiguous() ? out : at::empty_like(out, at::MemoryFormat::Contiguous);
  B200_KERNEL_CHECK(b200_arange(dst.data_ptr(), to_b200_dtype(t), n, s, st, scope.stream()));
  if (!dst.is_same(out)) out.copy_(dst);
  return out;
}
Tensor& k_arange_start_out(const at::Scalar& start, const at::Scalar& end, const at::Scalar& step, Tensor& out) {
  B200_DISPATCH("arange.start_out", (void)arange_out_device(start, end, step, out), (void)B200_CPU(arange_start_out, start, end, step, out));
  return out;
}

Tensor tri_device(const Tensor& self, int64_t k, bool upper) {
  TORCH_CHECK(self.dim() >= 2, "tril / triu: input must have at least 2 dimensions");
  OpScope scope(upper ? "triu" : "tril", self);
  Tensor x = self.contiguous();
  Tensor out = empty_b200(x.sizes(), x.scalar_type(), x.device().index());
  const int64_t rows = x.size(-2), cols = x.size(-1);
  const int64_t batch = rows * cols ? x.numel() / (rows * cols) : 0;
  B200_KERNEL_CHECK(b200_tri(x.data_ptr(), out.data_ptr(), (int)x.element_size(), batch, rows, cols, k, upper ? 1 : 0, scope.stream()));
  return out;
}
Tensor k_tril(const Tensor& self, int64_t k) { return B200_DISPATCH("tril", tri_device(self, k, false), B200_CPU(tril, self, k)); }
Tensor k_triu(const Tensor& self, int64_t k) { return B200_DISPATCH("triu", tri_device(self, k, true), B200_CPU(triu, self, k)); }
Tensor& k_tril_(Tensor& self, int64_t k) { self.copy_(k_tril(self, k)); return self; }
Tensor& k_triu_(Tensor& self, int64_t k) { self.copy_(k_triu(self, k)); return self; }

// ---- sort / topk -------------------------------------------------------------------------
std::tuple<Tensor, Tensor> sort_rows_device(const Tensor& self, int64_t dim, bool descending, int64_t k, const char* name) {
  const auto t = self.scalar_type();
  TORCH_CHECK(to_b200_dtype(t) >= 0 && !self.is_complex(), "b200 ", name, ": dtype ", t, " has no device kernel");
  Tensor x0 = self.dim() == 0 ? self.unsqueeze(0) : self;
  dim = at::maybe_wrap_dim(dim, x0.dim());
  const int64_t len = x0.size(dim);
  if (k < 0) k = len;
  TORCH_CHECK(k <= len, name, ": k out of range");
  OpScope scope(name, self);
  Tensor x = x0.movedim(dim, -1).contiguous();
  std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
  shape.back() = k;
  Tensor values = empty_b200(shape, t, self.device().index());
  Tensor indices = empty_b200(shape, at::kLong, self.device().index());
  const int64_t rows = len ? x.numel() / len : 0;
  // short rows of types that fit a float key: one shared-memory bitonic sort per row; everything else
  // (long rows, 64-bit keys, integers that a float cannot hold): the multi-pass sort over a workspace
  const bool small = len <= b200_sort_rows_max_len() && (float_type(t) || t == at::kByte || t == at::kChar || t == at::kBool);
  if (rows > 0 && k > 0) {
    if (small) {
      B200_KERNEL_CHECK(b200_sort_rows(x.data_ptr(), to_b200_dtype(t), (int)x.element_size(), rows, (int)len, descending ? 1 : 0, (int)k,
                                       values.data_ptr(), i64ptr(indices), scope.stream()));
    } else {
      Workspace ws((size_t)b200_sort_long_workspace_bytes(rows, len), scope);
      B200_KERNEL_CHECK(b200_sort_long(x.data_ptr(), to_b200_dtype(t), (int)x.element_size(), rows, len, descending ? 1 : 0, k,
                                       values.data_ptr(), i64ptr(indices), ws.get(), scope.stream()));
    }
  }
  values = values.movedim(-1, dim).contiguous();  // contiguous results, as from the stock kernels
  indices = indices.movedim(-1, dim).contiguous();
  if (self.dim() == 0) return {values.squeeze(0), indices.squeeze(0)};
  return {values, indices};
}
std::tuple<Tensor, Tensor> k_sort_stable(const Tensor& self, std::optional<bool> stable, int64_t dim, bool descending) {
  return B200_DISPATCH("sort.stable", sort_rows_device(self, dim, descending, -1, "sort"),
                       B200_CPU(sort_stable, self, stable, dim, descending));
}
std::tuple<Tensor, Tensor> k_sort(const Tensor& self, int64_t dim, bool descending) {
  return k_sort_stable(self, false, dim, descending);
}
std::tuple<Tensor, Tensor> k_topk(const Tensor& self, c10::SymInt k, int64_t dim, bool largest, bool sorted) {
  return B200_DISPATCH("topk", sort_rows_device(self, dim, largest, k.expect_int(), "topk"),
                       B200_CPU_SYMINT(topk, self, k, dim, largest, sorted));
}

// ---- 2-D resampling ---------------------------------------------------------------------
double resample_scale(int64_t in, int64_t out, std::optional<double> scale, bool align) {
  if (align) return out > 1 ? (double)(in - 1) / (double)(out - 1) : 0.0;
  return (scale.has_value() && *scale > 0) ? 1.0 / *scale : (double)in / (double)out;
}
Tensor resample_fwd(const Tensor& input, at::IntArrayRef osize, bool align, std::optional<double> sh, std::optional<double> sw, int mode) {
  TORCH_CHECK(input.dim() == 4 && osize.size() == 2 && float_type(input.scalar_type()), "b200 upsample: 4-D floating input expected");
  OpScope scope(mode ? "upsample_bilinear2d" : "upsample_nearest2d", input);
  const auto mf = input.suggest_memory_format();
  Tensor out = empty_b200({input.size(0), input.size(1), osize[0], osize[1]}, input.scalar_type(), input.device().index(), mf);
  long long sizes[6] = {input.size(0), input.size(1), input.size(2), input.size(3), osize[0], osize[1]};
  auto is = ll(input.strides()), os = ll(out.strides());
  B200_KERNEL_CHECK(b200_resample2d(input.data_ptr(), out.data_ptr(), to_b200_dtype(input.scalar_type()), sizes, is.data(), os.data(),
                                    resample_scale(input.size(2), osize[0], sh, align), resample_scale(input.size(3), osize[1], sw, align),
                                    align ? 1 : 0, mode, 0, nullptr, scope.stream()));
  return out;
}
Tensor resample_bwd(const Tensor& grad, at::IntArrayRef osize, at::IntArrayRef isize, bool align, std::optional<double> sh,
                    std::optional<double> sw, int mode) {
  TORCH_CHECK(grad.dim() == 4 && isize.size() == 4 && float_type(grad.scalar_type()), "b200 upsample backward: 4-D floating gradient expected");
  OpScope scope(mode ? "upsample_bilinear2d_backward" : "upsample_nearest2d_backward", grad);
  Tensor acc = at::zeros({isize[0], isize[1], isize[2], isize[3]}, grad.options().dtype(at::kFloat));
  long long sizes[6] = {isize[0], isize[1], isize[2], isize[3], osize[0], osize[1]};
  auto gs = ll(grad.strides());
  B200_KERNEL_CHECK(b200_resample2d(nullptr, const_cast<void*>(grad.const_data_ptr()), to_b200_dtype(grad.scalar_type()), sizes, nullptr,
                                    gs.data(), resample_scale(isize[2], osize[0], sh, align), resample_scale(isize[3], osize[1], sw, align),
                                    align ? 1 : 0, mode, 1, acc.data_ptr<float>(), scope.stream()));
  Tensor out = grad.scalar_type() == at::kFloat ? acc : acc.to(grad.scalar_type());
  return grad.suggest_memory_format() == at::MemoryFormat::ChannelsLast ? out.contiguous(at::MemoryFormat::ChannelsLast) : out;
}
Tensor k_upsample_nearest2d(const Tensor& self, c10::SymIntArrayRef osize, std::optional<double> sh, std::optional<double> sw) {
  auto os = C10_AS_INTARRAYREF_SLOW(osize);
  return B200_DISPATCH("upsample_nearest2d", resample_fwd(self, os, false, sh, sw, 0),
                       B200_CPU_SYMINT(upsample_nearest2d, self, osize, sh, sw));
}
Tensor k_upsample_nearest2d_backward(const Tensor& grad, c10::SymIntArrayRef osize, c10::SymIntArrayRef isize, std::optional<double> sh,
                                     std::optional<double> sw) {
  auto os = C10_AS_INTARRAYREF_SLOW(osize);
  auto is = C10_AS_INTARRAYREF_SLOW(isize);
  return B200_DISPATCH("upsample_nearest2d_backward", resample_bwd(grad, os, is, false, sh, sw, 0),
                       B200_CPU_SYMINT(upsample_nearest2d_backward, grad, osize, isize, sh, sw));
}
Tensor k_upsample_bilinear2d(const Tensor& self, c10::SymIntArrayRef osize, bool align, std::optional<double> sh, std::optional<double> sw) {
  auto os = C10_AS_INTARRAYREF_SLOW(osize);
  return B200_DISPATCH("upsample_bilinear2d", resample_fwd(self, os, align, sh, sw, 1),
                       B200_CPU_SYMINT(upsample_bilinear2d, self, osize, align, sh, sw));
}
Tensor k_upsample_bilinear2d_backward(const Tensor& grad, c10::SymIntArrayRef osize, c10::SymIntArrayRef isize, bool align,
                                      std::optional<double> sh, std::optional<double> sw) {
  auto os = C10_AS_INTARRAYREF_SLOW(osize);
  auto is = C10_AS_INTARRAYREF_SLOW(isize);
  return B200_DISPATCH("upsample_bilinear2d_backward", resample_bwd(grad, os, is, align, sh, sw, 1),
                       B200_CPU_SYMINT(upsample_bilinear2d_backward, grad, osize, isize, align, sh, sw));
}

// ---- NMS -----------------------------------------------------------------------------------
// Returns the indices of the boxes that survive, in order of descending score.
Tensor nms(const Tensor& boxes, const Tensor& scores, double iou_threshold) {
  check_same_device("nms", boxes, scores);
  TORCH_CHECK(boxes.dim() == 2 && boxes.size(1) == 4 && scores.dim() == 1 && scores.size(0) == boxes.size(0),
              "nms: boxes must be [N, 4] and scores [N]");
  const int64_t n = boxes.size(0);
  if (n == 0) return at::empty({0}, boxes.options().dtype(at::kLong));
  if (use_cpu_path() || !is_b200(boxes)) {
    // reference implementation on the host
    Tensor b = boxes.to(at::kCPU, at::kFloat).contiguous(), order = std::get<1>(scores.to(at::kCPU, at::kFloat).sort(0, true));
    auto bp = b.accessor<float, 2>();
    auto op = order.accessor<int64_t, 1>();
    std::vector<char> dead(n, 0);
    std::vector<int64_t> keep;
    for (int64_t a = 0; a < n; ++a) {
      if (dead[a]) continue;
      const int64_t i = op[a];
      keep.push_back(i);
      const float ai = (bp[i][2] - bp[i][0]) * (bp[i][3] - bp[i][1]);
      for (int64_t c = a + 1; c < n; ++c) {
        if (dead[c]) continue;
        const int64_t j = op[c];
        const float w = std::max(std::min(bp[i][2], bp[j][2]) - std::max(bp[i][0], bp[j][0]), 0.f);
        const float h = std::max(std::min(bp[i][3], bp[j][3]) - std::max(bp[i][1], bp[j][1]), 0.f);
        const float inter = w * h, aj = (bp[j][2] - bp[j][0]) * (bp[j][3] - bp[j][1]);
        if (inter > iou_threshold * (ai + aj - inter)) dead[c] = 1;
      }
    }
    return at::tensor(keep, at::kLong).to(boxes.device());
  }
  OpScope scope("nms", boxes);
  Tensor order = std::get<1>(scores.to(at::kFloat).sort(0, /*descending=*/true));
  Tensor sorted = boxes.to(at::kFloat).index_select(0, order).contiguous();
  const int64_t cb = (n + 63) / 64;
  Tensor mask = at::zeros({n, cb}, boxes.options().dtype(at::kLong));
  B200_KERNEL_CHECK(b200_nms_mask(sorted.data_ptr<float>(), (int)n, (float)iou_threshold,
                                  reinterpret_cast<unsigned long long*>(mask.data_ptr<int64_t>()), scope.stream()));
  // the greedy pass over the bit matrix is sequential; it runs on the host
  Tensor mask_h = mask.to(at::kCPU), order_h = order.to(at::kCPU);
  const uint64_t* mp = reinterpret_cast<const uint64_t*>(mask_h.data_ptr<int64_t>());
  const int64_t* op = order_h.data_ptr<int64_t>();
  std::vector<uint64_t> removed(cb, 0);
  std::vector<int64_t> keep;
  for (int64_t i = 0; i < n; ++i) {
    if (removed[i / 64] & (1ull << (i % 64))) continue;
    keep.push_back(op[i]);
    for (int64_t j = i / 64; j < cb; ++j) removed[j] |= mp[i * cb + j];
  }
  return at::tensor(keep, at::kLong).to(boxes.device());
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("gather", TORCH_FN(k_gather));
  m.impl("scatter.src", TORCH_FN(k_scatter_src));
  m.impl("scatter_.src", TORCH_FN(k_scatter_src_));
  m.impl("scatter.value", TORCH_FN(k_scatter_value));
  m.impl("scatter_.value", TORCH_FN(k_scatter_value_));
  m.impl("scatter_add", TORCH_FN(k_scatter_add));
  m.impl("scatter_add_", TORCH_FN(k_scatter_add_));
  m.impl("nonzero", TORCH_FN(k_nonzero));
  m.impl("masked_select", TORCH_FN(k_masked_select));
  m.impl("index.Tensor", TORCH_FN(k_index));
  m.impl("_index_put_impl_", TORCH_FN(k_index_put_impl_));
  m.impl("arange.start_out", TORCH_FN(k_arange_start_out));
  m.impl("tril", TORCH_FN(k_tril));
  m.impl("triu", TORCH_FN(k_triu));
  m.impl("tril_", TORCH_FN(k_tril_));
  m.impl("triu_", TORCH_FN(k_triu_));
  m.impl("sort", TORCH_FN(k_sort));
  m.impl("sort.stable", TORCH_FN(k_sort_stable));
  m.impl("topk", TORCH_FN(k_topk));
  m.impl("upsample_nearest2d", TORCH_FN(k_upsample_nearest2d));
  m.impl("upsample_nearest2d_backward", TORCH_FN(k_upsample_nearest2d_backward));
  m.impl("upsample_bilinear2d", TORCH_FN(k_upsample_bilinear2d));
  m.impl("upsample_bilinear2d_backward", TORCH_FN(k_upsample_bilinear2d_backward));
}

TORCH_LIBRARY_FRAGMENT(catch_b200, m) {
  // boxes [N, 4] as (x1, y1, x2, y2), scores [N]; returns the kept indices by descending score
  m.def("nms(Tensor boxes, Tensor scores, float iou_threshold) -> Tensor");
}
TORCH_LIBRARY_IMPL(catch_b200, CompositeExplicitAutograd, m) { m.impl("nms", TORCH_FN(nms)); }
// torchvision.ops.nms on this device (torchvision defines the schema when it is imported)
TORCH_LIBRARY_IMPL(torchvision, PrivateUse1, m) { m.impl("nms", TORCH_FN(nms)); }

}  // namespace ops
}  // namespace catch_b200
