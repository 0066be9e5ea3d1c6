#include "kernels.h"

#include <atomic>

namespace catch_b200 {
namespace ops {

static std::atomic<long long> g_launches{0};
void note_kernel_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
long long kernel_launch_count() { return g_launches.load(); }
void reset_kernel_launch_count() { g_launches.store(0); }

static int compute_class(at::ScalarType t) {
  if (t == at::kDouble) return 1;
  if (c10::isFloatingType(t)) return 0;
  return 2;
}

void launch_ew(at::TensorIteratorBase& iter, int op, double s0, double s1, void* stream,
               std::optional<at::ScalarType> compute) {
  if (iter.numel() == 0) return;
  TORCH_CHECK(iter.ndim() <= B200_EW_MAX_DIMS, "b200 elementwise: more than ", B200_EW_MAX_DIMS,
              " non-coalescable dimensions");
  TORCH_CHECK(iter.ntensors() <= B200_EW_MAX_OPERANDS, "b200 elementwise: too many operands");
  B200EwDesc d;
  std::memset(&d, 0, sizeof(d));
  d.op = op;
  d.ndim = iter.ndim();
  d.noperands = iter.ntensors();
  d.numel = iter.numel();
  d.scalar[0] = s0;
  d.scalar[1] = s1;
  for (int k = 0; k < d.ndim; ++k) d.shape[k] = iter.shape()[k];
  // Compute type: the promoted input dtype (comparisons promote inputs but
  // write bool); iterators built without promotion pass it explicitly.
  at::ScalarType ct = compute.has_value() ? *compute : iter.common_dtype();
  d.compute = compute_class(ct);
  bool dense = iter.ndim() <= 1;
  for (int i = 0; i < d.noperands; ++i) {
    d.dtype[i] = to_b200_dtype(iter.dtype(i));
    if (i > 0 && iter.is_cpu_scalar(i)) {
      d.scalar_mask |= 1 << i;
      d.scalar_operand[i] = iter.scalar_value<double>(i);
      d.ptr[i] = nullptr;
      continue;
    }
    TORCH_CHECK(iter.device(i).type() == c10::DeviceType::PrivateUse1, "b200 elementwise: operand ", i, " is on ",
                iter.device(i));
    d.ptr[i] = iter.data_ptr(i);
    const int64_t es = static_cast<int64_t>(iter.element_size(i));
    for (int k = 0; k < d.ndim; ++k) {
      const int64_t sb = iter.strides(i)[k];
      TORCH_CHECK(sb % es == 0, "b200 elementwise: byte stride not a multiple of the element size");
      d.strides[i][k] = sb / es;
    }
    if (d.ndim == 1 && d.strides[i][0] != 1) dense = false;
  }
  d.contiguous = dense ? 1 : 0;
  B200_KERNEL_CHECK(b200_elementwise(&d, stream));
}

void launch_copy(const at::Tensor& src, const at::Tensor& dst, void* stream) {
  if (dst.numel() == 0) return;
  auto iter = at::TensorIteratorConfig()
                  .add_output(dst)
                  .add_const_input(src)
                  .resize_outputs(false)
                  .check_all_same_dtype(false)
                  .check_all_same_device(false)
                  .build();
  if (iter.ndim() > B200_EW_MAX_DIMS) {
    // Too many irregular dimensions: densify the source first.
    at::Tensor dense = empty_b200(src.sizes(), src.scalar_type(), src.device().index());
    // recursion terminates: a dense destination coalesces with most sources
    launch_copy(src, dense, stream);
    launch_copy(dense, dst, stream);
    return;
  }
  // Value-preserving compute class: the wider of the two dtypes' classes.
  const at::ScalarType ct = (src.scalar_type() == at::kDouble || dst.scalar_type() == at::kDouble) ? at::kDouble
                            : (c10::isFloatingType(src.scalar_type()) ? at::kFloat
                               : (c10::isFloatingType(dst.scalar_type()) && src.scalar_type() != at::kLong ? at::kFloat
                                                                                                       : at::kLong));
  launch_ew(iter, EW_COPY, 0, 0, stream, ct);
}

void launch_fill(const at::Tensor& dst, double value, void* stream) {
  if (dst.numel() == 0) return;
  auto iter = at::TensorIteratorConfig().add_output(dst).resize_outputs(false).check_all_same_dtype(false).build();
  launch_ew(iter, EW_FILL, value, 0, stream, dst.scalar_type());
}

}  // namespace ops
}  // namespace catch_b200
