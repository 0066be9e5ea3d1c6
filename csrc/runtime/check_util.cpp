#include "check_util.h"

#include <cmath>
#include <cstring>

#include "log.h"

namespace catch_b200 {

namespace {
at::Tensor as_double_cpu(const at::Tensor& t) { return t.detach().to(at::kCPU).to(at::kDouble); }
}  // namespace

TensorDiff tensorDiff(const at::Tensor& a_in, const at::Tensor& b_in) {
  TORCH_CHECK(a_in.sizes() == b_in.sizes(), "tensor sizes differ: ", a_in.sizes(), " vs ", b_in.sizes());
  TensorDiff d;
  if (a_in.numel() == 0) return d;
  const at::Tensor a = as_double_cpu(a_in), b = as_double_cpu(b_in);
  const at::Tensor diff = (a - b).abs();
  d.max_abs = diff.max().item<double>();
  const double sq = diff.pow(2).sum().item<double>();
  // tiny references: compare against a floor so that noise around zero does not read as a large relative error
  const double eps = 1.0 / 16384;
  double ref_sq = a.pow(2).sum().item<double>();
  if (ref_sq <= eps) ref_sq += eps;
  d.rel_rms = sq <= 4 * eps * eps ? 0.0 : std::sqrt(sq / ref_sq);
  const double abs_sum = a.abs().sum().item<double>();
  d.rel_abs = abs_sum == 0.0 ? (diff.sum().item<double>() == 0.0 ? 0.0 : INFINITY) : diff.sum().item<double>() / abs_sum;
  const double ma = a.abs().mean().item<double>(), mb = b.abs().mean().item<double>();
  d.rel_mean = ma == 0.0 ? (mb == 0.0 ? 0.0 : INFINITY) : (ma - mb) / ma;
  return d;
}

void assertTensorsEqual(const at::Tensor& a, const at::Tensor& b, double prec, bool use_MSE, bool use_RAE, bool use_RMA) {
  const TensorDiff d = tensorDiff(a, b);
  const char* what = use_MSE ? "relative RMS error" : use_RAE ? "relative absolute error" : use_RMA ? "relative mean error"
                                                                                                     : "maximum absolute error";
  const double v = use_MSE ? d.rel_rms : use_RAE ? d.rel_abs : use_RMA ? d.rel_mean : d.max_abs;
  TORCH_CHECK(v <= prec, "tensors differ: ", what, " ", v, " is above the bound ", prec);
}

int64_t batchCheckErrors(const at::Tensor& infos, const char* name, bool allow_singular) {
  const at::Tensor h = infos.detach().to(at::kCPU).to(at::kInt).contiguous().view({-1});
  const int* p = h.data_ptr<int>();
  int64_t failed = 0;
  for (int64_t i = 0; i < h.numel(); ++i) {
    const int info = p[i];
    if (info == 0) continue;
    if (info < 0) {
      B200LOG(ERROR) << name << ": batch " << i << ": argument " << -info << " had an illegal value";
      ++failed;
    } else if (std::strstr(name, "svd")) {
      B200LOG(ERROR) << name << ": batch " << i << ": the SVD did not converge (code " << info << "); results may be imprecise";
      ++failed;
    } else if (std::strstr(name, "symeig") || std::strstr(name, "eigh")) {
      B200LOG(ERROR) << name << ": batch " << i << ": the eigen-solver did not converge; " << info
                     << " off-diagonal elements of the intermediate tridiagonal form stayed non-zero";
      ++failed;
    } else if (!allow_singular) {
      B200LOG(ERROR) << name << ": batch " << i << ": U(" << info << "," << info << ") is zero: the factor is singular";
      ++failed;
    }
  }
  return failed;
}

}  // namespace catch_b200
