// TensorImpl of the b200 device plus construction helpers.
//
// The reference's MLUTensorImpl (torch_mlu/csrc/aten/core/tensor_impl.h:47-212)
// carries a shadow CPU storage, an on-chip dtype and a view-op recorder because
// its device had no strides and no 64-bit types.  B200 memory holds real strided
// tensors, so this subclass is thin: it only carries optional backend metadata
// that producers attach for consumers (per-channel sum / sum-of-squares written
// by the convolution epilogue so the following batch norm can skip its
// statistics pass).
#pragma once
#include <ATen/ATen.h>
#include <c10/core/TensorImpl.h>
#include <memory>
#include "queue.h"

namespace catch_b200 {

// Per-channel statistics a producer kernel computed as a by-product.
struct ChannelStats {
  at::Tensor sum;      // fp32 [C]
  at::Tensor sumsq;    // fp32 [C]
  int64_t count = 0;   // elements per channel
  uint32_t version = 0;  // tensor version when attached
};

class B200TensorImpl final : public c10::TensorImpl {
 public:
  B200TensorImpl(c10::Storage&& storage, c10::DispatchKeySet ks, const caffe2::TypeMeta dtype)
      : c10::TensorImpl(std::move(storage), ks, dtype) {}

  c10::intrusive_ptr<c10::TensorImpl> shallow_copy_and_detach(const c10::VariableVersion& vc,
                                                              bool allow_tensor_metadata_change) const override;
  c10::intrusive_ptr<c10::TensorImpl> shallow_copy_and_detach(c10::VariableVersion&& vc,
                                                              bool allow_tensor_metadata_change) const override;
  void shallow_copy_from(const c10::intrusive_ptr<c10::TensorImpl>& impl) override;

  std::shared_ptr<ChannelStats> channel_stats;

 private:
  template <typename VC>
  c10::intrusive_ptr<c10::TensorImpl> detach_core(VC&& vc, bool allow_tensor_metadata_change) const {
    auto impl = c10::make_intrusive<B200TensorImpl>(c10::Storage(storage()), key_set(), dtype());
    copy_tensor_metadata(this, impl.get(), std::forward<VC>(vc), allow_tensor_metadata_change);
    impl->channel_stats = channel_stats;
    impl->refresh_numel();
    impl->refresh_contiguous();
    return impl;
  }
  const char* tensorimpl_type_name() const override { return "B200TensorImpl"; }
};

inline B200TensorImpl* maybe_b200_impl(const at::Tensor& t) {
  return dynamic_cast<B200TensorImpl*>(t.unsafeGetTensorImpl());
}

// Allocation through the caching allocator on the current queue of `device`.
at::Tensor empty_b200(c10::IntArrayRef size, c10::ScalarType dtype, int device,
                      std::optional<c10::MemoryFormat> mf = std::nullopt);
at::Tensor empty_strided_b200(c10::IntArrayRef size, c10::IntArrayRef stride, c10::ScalarType dtype, int device);
inline bool is_b200(const at::Tensor& t) { return t.defined() && t.device().type() == c10::DeviceType::PrivateUse1; }

}  // namespace catch_b200
