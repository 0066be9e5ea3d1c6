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
void run_gemm(const Tensor& a, const Tensor& b, Tensor& out, const Tensor* bias, const Tensor* res, double alpha,
              double beta, int act) {
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
Tensor b200_bmm(const Tensor& a, const Tensor& b) { return B200_DISPATCH("bmm", bmm_device(a, b), B200_CPU(bmm, a, b)); }
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
  return B200_DISPATCH("baddbmm", baddbmm_device(self, a, b, beta, alpha), B200_CPU(baddbmm, self, a, b, beta, alpha));
}

}  // namespace

// Fused linear used by the fusion pass and the quantization-free fast path:
// act(x @ w^T + bias); x [.., K], w [N, K].
at::Tensor linear_act(const at::Tensor& x, const at::Tensor& w, const std::optional<at::Tensor>& bias, int64_t act) {
  TORCH_CHECK(x.size(-1) == w.size(1), "linear_act: shape mismatch");
  auto x2 = x.reshape({-1, x.size(-1)});
  std::vector<int64_t> osz(x.sizes().begin(), x.sizes().end());
  osz.back() = w.size(0);
  if (use_cpu_path() || !gemm_dtype_ok(x.scalar_type()) || x.scalar_type() != w.scalar_type()) {
    at::Tensor y = at::linear(x, w, bias);
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
