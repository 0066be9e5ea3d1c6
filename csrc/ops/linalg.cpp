// mm / addmm / bmm / baddbmm on the tcgen05 GEMM kernel.
//
// Parity: torch_mlu/csrc/aten/operators/cnnl/{matmul,addmm,bmm}.cpp.  Like the
// reference (internal_util.cpp:226-270) transposed views are not materialised:
// the operand's major-ness is derived from its strides and handed to the
// kernel's tensor-map / descriptor setup.
#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Scalar;
using at::Tensor;

bool gemm_dtype_ok(at::ScalarType t) { return t == at::kBFloat16 || t == at::kHalf || t == at::kFloat; }

struct Operand {
  Tensor t;        // keeps a possible copy alive
  int64_t ld = 0;  // elements
  int mn_major = 0;
  int64_t batch_stride = 0;
};

// `rows` indexes the M (or N) dimension, `k` the reduction dimension of a 2-D
// (or batched 3-D) view.
Operand prep(const Tensor& x, int64_t rows_dim, int64_t k_dim) {
  const int64_t es = x.element_size();
  auto aligned = [&](const Tensor& t, int64_t ld, int64_t bs) {
    return (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0) && (ld * es) % 16 == 0 && (bs * es) % 16 == 0 && ld > 0;
  };
  const int64_t bs = x.dim() == 3 ? x.stride(0) : 0;
  Operand o;
  if (x.stride(k_dim) == 1 && x.size(k_dim) > 1 && aligned(x, x.stride(rows_dim), bs) &&
      x.stride(rows_dim) >= x.size(k_dim)) {
    o.t = x; o.ld = x.stride(rows_dim); o.mn_major = 0; o.batch_stride = bs;
    return o;
  }
  if (es == 2 && x.stride(rows_dim) == 1 && x.size(rows_dim) > 1 && aligned(x, x.stride(k_dim), bs) &&
      x.stride(k_dim) >= x.size(rows_dim)) {
    o.t = x; o.ld = x.stride(k_dim); o.mn_major = 1; o.batch_stride = bs;
    return o;
  }
  // Irregular strides: copy into a K-major buffer whose row pitch is 16-byte aligned.
  const int64_t rows = x.size(rows_dim), k = x.size(k_dim);
  const int64_t per16 = 16 / es;
  const int64_t ld = (k + per16 - 1) / per16 * per16;
  const int64_t nb = x.dim() == 3 ? x.size(0) : 1;
  Tensor buf = empty_b200({nb, rows, ld}, x.scalar_type(), x.device().index());
  Tensor view = buf.narrow(2, 0, k);
  Tensor src = x.dim() == 3 ? x : x.unsqueeze(0);
  if (rows_dim > k_dim) src = src.transpose(1, 2);
  view.copy_(src);
  o.t = buf; o.ld = ld; o.mn_major = 0; o.batch_stride = rows * ld;
  return o;
}

// out[b, M, N] = act(alpha * a @ b + bias + beta * res)
// accumulate: out is fp32 and receives out += alpha * a @ b (K may be split among CTAs)
void run_gemm(const Tensor& a, const Tensor& b, Tensor& out, const Tensor* bias, const Tensor* res, double alpha,
              double beta, int act, bool accumulate = false) {
  const bool batched = a.dim() == 3;
  const int64_t M = a.size(-2), K = a.size(-1), N = b.size(-1);
  OpScope scope("gemm", out);
  Operand A = prep(a, batched ? 1 : 0, batched ? 2 : 1);
  Operand B = prep(b, batched ? 2 : 1, batched ? 1 : 0);
  B200GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = batched ? (int)a.size(0) : 1;
  p.A = A.t.data_ptr(); p.B = B.t.data_ptr(); p.D = out.data_ptr();
  p.lda = A.ld; p.ldb = B.ld; p.ldd = N;
  p.stride_a = A.batch_stride; p.stride_b = B.batch_stride; p.stride_d = M * N;
  p.a_mn_major = A.mn_major; p.b_mn_major = B.mn_major;
  p.ab_dtype = to_b200_dtype(a.scalar_type());
  p.d_dtype = to_b200_dtype(out.scalar_type());
  if (bias) {
    p.bias = bias->data_ptr();
    p.bias_dtype = to_b200_dtype(bias->scalar_type());
  }
  if (res) {
    p.residual = res->data_ptr();
    p.ldr = res->dim() >= 2 ? res->stride(-2) : 0;
    p.stride_r = res->dim() == 3 ? res->stride(0) : 0;
    p.res_dtype = to_b200_dtype(res->scalar_type());
  }
  p.alpha = (float)alpha; p.beta = (float)beta; p.act = act;
  p.accumulate = accumulate ? 1 : 0;
  B200_KERNEL_CHECK(b200_gemm(&p, scope.stream()));
}

void check_mm(const Tensor& a, const Tensor& b) {
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "mm: both arguments must be 2-D, got ", a.dim(), "-D and ", b.dim(), "-D");
  TORCH_CHECK(a.size(1) == b.size(0), "mat1 and mat2 shapes cannot be multiplied (", a.size(0), "x", a.size(1), " and ",
              b.size(0), "x", b.size(1), ")");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "expected m1 and m2 to have the same dtype, but got: ",
              a.scalar_type(), " != ", b.scalar_type());
}

Tensor mm_device(const Tensor& a, const Tensor& b) {
  check_mm(a, b);
  Tensor out = empty_b200({a.size(0), b.size(1)}, a.scalar_type(), a.device().index());
  if (out.numel() == 0) return out;
  if (a.size(1) == 0) return out.zero_();
  TORCH_CHECK(gemm_dtype_ok(a.scalar_type()), "b200 mm: unsupported dtype ", a.scalar_type());
  run_gemm(a, b, out, nullptr, nullptr, 1.0, 0.0, 0);
  return out;
}
Tensor b200_mm(const Tensor& a, const Tensor& b) {
  check_same_device("mm", a, b);
  return B200_DISPATCH("mm", mm_device(a, b), B200_CPU(mm, a, b));
}
Tensor& mm_out(const Tensor& a, const Tensor& b, Tensor& out) {
  Tensor r = b200_mm(a, b);
  out.resize_(r.sizes());
  out.copy_(r);
  return out;
}

Tensor addmm_device(const Tensor& self, const Tensor& m1, const Tensor& m2, const Scalar& beta, const Scalar& alpha) {
  check_mm(m1, m2);
  TORCH_CHECK(gemm_dtype_ok(m1.scalar_type()), "b200 addmm: unsupported dtype ", m1.scalar_type());
  const int64_t M = m1.size(0), N = m2.size(1);
  Tensor out = empty_b200({M, N}, m1.scalar_type(), m1.device().index());
  if (out.numel() == 0) return out;
  const double be = beta.toDouble(), al = alpha.toDouble();
  if (m1.size(1) == 0) {
    out.copy_(self.expand({M, N}));
    return out.mul_(be);
  }
  const bool as_bias = be == 1.0 && (self.dim() == 1 || (self.dim() == 2 && self.size(0) == 1)) &&
                       self.size(-1) == N && self.stride(-1) == 1;
  if (as_bias) {
    run_gemm(m1, m2, out, &self, nullptr, al, 0.0, 0);
  } else if (be == 0.0) {
    run_gemm(m1, m2, out, nullptr, nullptr, al, 0.0, 0);
  } else {
    Tensor r = self.expand({M, N});
    if (r.stride(1) != 1) r = r.contiguous();
    run_gemm(m1, m2, out, nullptr, &r, al, be, 0);
  }
  return out;
}
Tensor b200_addmm(const Tensor& self, const Tensor& m1, const Tensor& m2, const Scalar& beta, const Scalar& alpha) {
  check_same_device("addmm", m1, m2, self);
  return B200_DISPATCH("addmm", addmm_device(self, m1, m2, beta, alpha), B200_CPU(addmm, self, m1, m2, beta, alpha));
}
Tensor& addmm_out(const Tensor& self, const Tensor& m1, const Tensor& m2, const Scalar& beta, const Scalar& alpha,
                  Tensor& out) {
  Tensor r = b200_addmm(self, m1, m2, beta, alpha);
  out.resize_(r.sizes());
  out.copy_(r);
  return out;
}
Tensor& addmm_(Tensor& self, const Tensor& m1, const Tensor& m2, const Scalar& beta, const Scalar& alpha) {
  Tensor r = b200_addmm(self, m1, m2, beta, alpha);
  self.copy_(r);
  return self;
}

Tensor bmm_device(const Tensor& a, const Tensor& b) {
  TORCH_CHECK(a.dim() == 3 && b.dim() == 3, "batch1 and batch2 must be 3D tensors");
  TORCH_CHECK(a.size(0) == b.size(0) && a.size(2) == b.size(1), "bmm: incompatible shapes ", a.sizes(), " and ", b.sizes());
  TORCH_CHECK(gemm_dtype_ok(a.scalar_type()) && a.scalar_type() == b.scalar_type(), "b200 bmm: unsupported dtype ", a.scalar_type());
  Tensor out = empty_b200({a.size(0), a.size(1), b.size(2)}, a.scalar_type(), a.device().index());
  if (out.numel() == 0) return out;
  if (a.size(2) == 0) return out.zero_();
  run_gemm(a, b, out, nullptr, nullptr, 1.0, 0.0, 0);
  return out;
}
Tensor b200_bmm(const Tensor& a, const Tensor& b) {
  check_same_device("bmm", a, b);
  return B200_DISPATCH("bmm", bmm_device(a, b), B200_CPU(bmm, a, b));
}
Tensor& bmm_out(const Tensor& a, const Tensor& b, Tensor& out) {
  Tensor r = b200_bmm(a, b);
  out.resize_(r.sizes());
  out.copy_(r);
  return out;
}
Tensor baddbmm_device(const Tensor& self, const Tensor& a, const Tensor& b, const Scalar& beta, const Scalar& alpha) {
  TORCH_CHECK(a.dim() == 3 && b.dim() == 3, "batch1 and batch2 must be 3D tensors");
  TORCH_CHECK(gemm_dtype_ok(a.scalar_type()), "b200 baddbmm: unsupported dtype ", a.scalar_type());
  Tensor out = empty_b200({a.size(0), a.size(1), b.size(2)}, a.scalar_type(), a.device().index());
  if (out.numel() == 0) return out;
  Tensor r = self.expand(out.sizes());
  if (r.stride(2) != 1) r = r.contiguous();
  if (beta.toDouble() == 0.0) run_gemm(a, b, out, nullptr, nullptr, alpha.toDouble(), 0.0, 0);
  else run_gemm(a, b, out, nullptr, &r, alpha.toDouble(), beta.toDouble(), 0);
  return out;
}
Tensor b200_baddbmm(const Tensor& self, const Tensor& a, const Tensor& b, const Scalar& beta, const Scalar& alpha) {
  check_same_device("baddbmm", a, b, self);
  return B200_DISPATCH("baddbmm", baddbmm_device(self, a, b, beta, alpha), B200_CPU(baddbmm, self, a, b, beta, alpha));
}

}  // namespace

// Fused linear used by the fusion pass and the quantization-free fast path:
// act(x @ w^T + bias); x [.., K], w [N, K].
at::Tensor linear_act(const at::Tensor& x, const at::Tensor& w, const std::optional<at::Tensor>& bias, int64_t act) {
  check_same_device("linear_act", x, w, bias);
  TORCH_CHECK(x.size(-1) == w.size(1), "linear_act: shape mismatch");
  auto x2 = x.reshape({-1, x.size(-1)});
  std::vector<int64_t> osz(x.sizes().begin(), x.sizes().end());
  osz.back() = w.size(0);
  if (use_cpu_path() || !gemm_dtype_ok(x.scalar_type()) || x.scalar_type() != w.scalar_type()) {
    // the fused kernel takes an fp32 bias next to 16-bit operands; the stock operator wants one dtype
    std::optional<at::Tensor> b = bias;
    if (b.has_value() && b->defined() && b->scalar_type() != x.scalar_type()) b = b->to(x.scalar_type());
    at::Tensor y = at::linear(x, w, b);
    if (act == 1) y = at::relu(y);
    else if (act == 2) y = at::gelu(y);
    return y;
  }
  at::Tensor out = empty_b200({x2.size(0), w.size(0)}, x.scalar_type(), x.device().index());
  if (out.numel()) {
    at::Tensor bt = w.t();
    const at::Tensor* bp = (bias.has_value() && bias->defined()) ? &*bias : nullptr;
    run_gemm(x2, bt, out, bp, nullptr, 1.0, 0.0, (int)act);
  }
  return out.reshape(osz);
}

// out[o, i] = alpha * a[o, i] @ b[o, i] over 4-D operands [B1, B2, M, K] x [B1, B2, K, N] with arbitrary batch strides:
// head-split views of [batch, seq, heads * dim] activations multiply without being copied into [batch * heads, ...]
// first, and `out` may itself be such a view (16-bit or, with accumulate, fp32 that is added to).
at::Tensor gemm_nd(const at::Tensor& a, const at::Tensor& b, const std::optional<at::Tensor>& out_opt, double alpha) {
  check_same_device("gemm_nd", a, b, out_opt);
  TORCH_CHECK(a.dim() == 4 && b.dim() == 4 && a.size(0) == b.size(0) && a.size(1) == b.size(1) && a.size(3) == b.size(2),
              "gemm_nd: expected [B1, B2, M, K] x [B1, B2, K, N], got ", a.sizes(), " and ", b.sizes());
  TORCH_CHECK(a.scalar_type() == b.scalar_type() && (a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf),
              "gemm_nd: 16-bit operands of one dtype expected");
  const int64_t B1 = a.size(0), B2 = a.size(1), M = a.size(2), K = a.size(3), N = b.size(3);
  at::Tensor out = (out_opt.has_value() && out_opt->defined()) ? *out_opt : empty_b200({B1, B2, M, N}, a.scalar_type(), a.device().index());
  TORCH_CHECK(out.dim() == 4 && out.size(0) == B1 && out.size(1) == B2 && out.size(2) == M && out.size(3) == N && out.stride(3) == 1,
              "gemm_nd: out must be [B1, B2, M, N] with a unit innermost stride");
  if (out.numel() == 0) return out;
  if (use_cpu_path()) {  // host path (host simulation, force-CPU mode): fp32 product, rounded once into `out`
    out.copy_(at::matmul(a.to(at::kFloat), b.to(at::kFloat)).mul_(alpha));
    return out;
  }
  TORCH_CHECK(is_b200(a), "gemm_nd: operands must be on the device");
  if (K == 0) return out.zero_();
  const int64_t es = 2;
  struct Op4 { at::Tensor t; int64_t ld; int mn; int64_t s1, s2; };
  auto prep4 = [&](const at::Tensor& x, int rows_dim, int k_dim) {
    auto ok = [&](int64_t ld) {
      return reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0 && (ld * es) % 16 == 0 && (x.stride(0) * es) % 16 == 0 &&
             (x.stride(1) * es) % 16 == 0 && ld > 0 && x.stride(0) > 0 && x.stride(1) > 0;
    };
    if (x.stride(k_dim) == 1 && x.size(k_dim) > 1 && ok(x.stride(rows_dim)) && x.stride(rows_dim) >= x.size(k_dim))
      return Op4{x, x.stride(rows_dim), 0, x.stride(1), x.stride(0)};
    if (x.stride(rows_dim) == 1 && x.size(rows_dim) > 1 && ok(x.stride(k_dim)) && x.stride(k_dim) >= x.size(rows_dim))
      return Op4{x, x.stride(k_dim), 1, x.stride(1), x.stride(0)};
    // irregular: a dense K-major copy with a 16-byte aligned row pitch
    const int64_t rows = x.size(rows_dim), k = x.size(k_dim), ld = (k + 7) / 8 * 8;
    at::Tensor buf = empty_b200({x.size(0), x.size(1), rows, ld}, x.scalar_type(), x.device().index());
    buf.narrow(3, 0, k).copy_(rows_dim > k_dim ? x.transpose(2, 3) : x);
    return Op4{buf, ld, 0, rows * ld, x.size(1) * rows * ld};
  };
  Op4 A = prep4(a, 2, 3), Bm = prep4(b, 3, 2);
  OpScope scope("gemm_nd", out);
  B200GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)(B1 * B2); p.batch_inner = (int)B2;
  p.A = A.t.data_ptr(); p.B = Bm.t.data_ptr(); p.D = out.data_ptr();
  p.lda = A.ld; p.ldb = Bm.ld; p.ldd = out.stride(2);
  p.stride_a = A.s1; p.stride_a2 = A.s2; p.stride_b = Bm.s1; p.stride_b2 = Bm.s2;
  p.stride_d = out.stride(1); p.stride_d2 = out.stride(0);
  p.a_mn_major = A.mn; p.b_mn_major = Bm.mn;
  p.ab_dtype = to_b200_dtype(a.scalar_type());
  p.d_dtype = to_b200_dtype(out.scalar_type());
  p.alpha = (float)alpha;
  B200_KERNEL_CHECK(b200_gemm(&p, scope.stream()));
  return out;
}

// Backward of y = x @ w^T + bias for 16-bit x / w whose master weight (and its gradient) are fp32:
//   dx = grad @ w                               (16-bit, like x)
//   dw = grad^T @ x  in fp32, K split over the GPU, added straight into `accum_w` (a flat fp32 [N * K] view of
//        the gradient bucket) when that is given, else returned as a new fp32 tensor;
//   db = column sums of grad in fp32, added into `accum_b` or returned.
// Undefined results stand for "not needed" or "added in place".
std::tuple<at::Tensor, at::Tensor, at::Tensor> linear_backward_fp32w(const at::Tensor& grad, const at::Tensor& x, const at::Tensor& w,
                                                                     bool need_dx, bool need_dw, bool need_db,
                                                                     const std::optional<at::Tensor>& accum_w,
                                                                     const std::optional<at::Tensor>& accum_b) {
  TORCH_CHECK(grad.scalar_type() == x.scalar_type() && x.scalar_type() == w.scalar_type() &&
                  (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf),
              "linear_backward_fp32w: 16-bit operands of one dtype expected");
  const int64_t N = w.size(0), K = w.size(1);
  if (use_cpu_path()) {  // host path (host simulation, force-CPU mode): the same three results from fp32 products
    at::Tensor gf = grad.reshape({-1, N}).to(at::kFloat), xf = x.reshape({-1, K}).to(at::kFloat);
    at::Tensor dx, dw, db;
    if (need_dx) dx = at::mm(gf, w.to(at::kFloat)).to(x.scalar_type()).reshape(x.sizes());
    if (need_dw) {
      dw = at::mm(gf.t(), xf);
      if (accum_w.has_value() && accum_w->defined()) {
        TORCH_CHECK(accum_w->scalar_type() == at::kFloat && accum_w->numel() == N * K && accum_w->is_contiguous(),
                    "linear_backward_fp32w: accum_w must be a contiguous fp32 tensor of the weight's size");
        accum_w->view({N, K}).add_(dw);
        dw = at::Tensor();
      }
    }
    if (need_db) {
      db = gf.sum(std::vector<int64_t>{0});
      if (accum_b.has_value() && accum_b->defined()) {
        accum_b->view({N}).add_(db);
        db = at::Tensor();
      }
    }
    return {dx, dw, db};
  }
  TORCH_CHECK(is_b200(grad), "linear_backward_fp32w: operands must be on the device");
  at::Tensor g2 = grad.reshape({-1, N}), x2 = x.reshape({-1, K});
  if (!g2.is_contiguous()) g2 = g2.contiguous();
  if (!x2.is_contiguous()) x2 = x2.contiguous();
  at::Tensor dx, dw, db;
  if (need_dx) {
    at::Tensor out = empty_b200({g2.size(0), K}, x.scalar_type(), x.device().index());
    if (out.numel()) run_gemm(g2, w, out, nullptr, nullptr, 1.0, 0.0, 0);
    dx = out.reshape(x.sizes());
  }
  if (need_dw) {
    const bool direct = accum_w.has_value() && accum_w->defined();
    at::Tensor acc;
    if (direct) {
      TORCH_CHECK(accum_w->scalar_type() == at::kFloat && accum_w->numel() == N * K && accum_w->is_contiguous(),
                  "linear_backward_fp32w: accum_w must be a contiguous fp32 tensor of the weight's size");
      acc = accum_w->view({N, K});
    } else {
      acc = at::zeros({N, K}, grad.options().dtype(at::kFloat));
    }
    if (g2.size(0) > 0) {
      at::Tensor gt = g2.t();
      // the reduce-add epilogue addresses the target through a tensor map: 16-byte aligned base and rows
      if (K % 4 == 0 && reinterpret_cast<uintptr_t>(acc.data_ptr()) % 16 == 0) {
        run_gemm(gt, x2, acc, nullptr, nullptr, 1.0, 0.0, 0, /*accumulate=*/true);
      } else {
        at::Tensor tmp = empty_b200({N, K}, at::kFloat, x.device().index());
        run_gemm(gt, x2, tmp, nullptr, nullptr, 1.0, 0.0, 0);
        acc.add_(tmp);
      }
    }
    if (!direct) dw = acc;
  }
  if (need_db) {
    at::Tensor s = g2.sum({0}, /*keepdim=*/false, at::kFloat);
    if (accum_b.has_value() && accum_b->defined()) const_cast<at::Tensor&>(*accum_b).view({N}).add_(s);
    else db = s;
  }
  return {dx, dw, db};
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  m.impl("mm", TORCH_FN(b200_mm));
  m.impl("mm.out", TORCH_FN(mm_out));
  m.impl("addmm", TORCH_FN(b200_addmm));
  m.impl("addmm.out", TORCH_FN(addmm_out));
  m.impl("addmm_", TORCH_FN(addmm_));
  m.impl("bmm", TORCH_FN(b200_bmm));
  m.impl("bmm.out", TORCH_FN(bmm_out));
  m.impl("baddbmm", TORCH_FN(b200_baddbmm));
}

}  // namespace ops
}  // namespace catch_b200
