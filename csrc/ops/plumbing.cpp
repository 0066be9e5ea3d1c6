// Tensor factories, views, copies and the boxed CPU fallback for the b200 device.
//
// Parity: OpMethods::empty / empty_strided (op_methods.cpp:71-125), cnnl_copy_
// (cnnl/copy.cpp:38-121: D2D, dtype-changing, H2D, D2H), the view family
// (alias/as_strided/set_storage/reshape...), _local_scalar_dense (scalar.cpp)
// and the boxed backend fallback mlu_wrapper
// (torch_mlu/tools/template/aten_mlu_type_default.cpp:44-314) of the reference.
#include <ATen/native/Resize.h>
#include <ATen/native/TensorShape.h>
#include <ATen/ops/_copy_from_and_resize_native.h>
#include <ATen/ops/as_strided_native.h>
#include <ATen/ops/view_native.h>
#include <ATen/ops/_reshape_alias_native.h>
#include <ATen/ops/unfold_native.h>
#include <c10/core/ScalarType.h>

#include <mutex>
#include <unordered_set>

#include "../runtime/host_allocator.h"
#include "common.h"
#include "../runtime/graph.h"
#include "../runtime/profiler.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {

// --------------------------------------------------------------------- OpScope
static int device_of_tensor(const at::Tensor& t) {
  return (t.defined() && is_b200(t)) ? t.device().index() : current_device();
}
OpScope::OpScope(const char* name, const at::Tensor& t) : OpScope(name, device_of_tensor(t)) {}
OpScope::OpScope(const char* name, int device) : name_(name), device_(device), sw_(device) {
  B200LOG(DBG) << "op " << name << " on b200:" << device;
  prev_op_ = trace_set_current_op(name);
}
OpScope::~OpScope() noexcept(false) {
  trace_set_current_op(prev_op_);
  if (flags().async_disable && !hostsim() && !graphCaptureActive()) getCurrentQueue(device_).synchronize();
}

std::string describe(const at::Tensor& t) {
  if (!t.defined()) return "undefined";
  std::ostringstream os;
  os << c10::toString(t.scalar_type()) << t.sizes() << "{" << t.strides() << "}@" << t.device();
  return os.str();
}

// -------------------------------------------------------------- boxed fallback
void cpu_fallback(const c10::OperatorHandle& op, torch::jit::Stack* stack) {
  const auto& name = op.schema().operator_name();
  if (!use_cpu_path()) {
    TORCH_CHECK_NOT_IMPLEMENTED(flags().fallback_to_cpu, "b200: operator '", c10::toString(name),
                                "' has no device kernel and the CPU fallback is disabled "
                                "(CATCH_B200_FALLBACK_TO_CPU=0).");
    static std::mutex mu;
    static std::unordered_set<std::string> seen;
    std::string key = c10::toString(name);
    bool first;
    {
      std::lock_guard<std::mutex> g(mu);
      first = seen.insert(key).second;
    }
    if (first) B200LOG(WARNING) << "operator '" << key << "' has no b200 kernel; it runs on the CPU (reported once).";
  } else {
    B200LOG(DBG) << "operator '" << c10::toString(name) << "' runs on the CPU path.";
  }
  at::native::cpu_fallback(op, stack);
}

// ------------------------------------------------------------------- factories
static at::Tensor empty_memory_format(c10::IntArrayRef size, std::optional<at::ScalarType> dtype,
                                      std::optional<at::Layout> layout, std::optional<at::Device> device,
                                      std::optional<bool> pin_memory, std::optional<at::MemoryFormat> mf) {
  TORCH_CHECK(!layout.has_value() || *layout == at::kStrided, "b200 tensors are strided only");
  TORCH_CHECK(!pin_memory.value_or(false), "Only dense CPU tensors can be pinned");
  const int dev = (device.has_value() && device->has_index()) ? device->index() : current_device();
  return empty_b200(size, dtype.value_or(at::get_default_dtype_as_scalartype()), dev, mf);
}

static at::Tensor b200_empty_strided(c10::IntArrayRef size, c10::IntArrayRef stride, std::optional<at::ScalarType> dtype,
                                std::optional<at::Layout> layout, std::optional<at::Device> device,
                                std::optional<bool> pin_memory) {
  TORCH_CHECK(!layout.has_value() || *layout == at::kStrided, "b200 tensors are strided only");
  TORCH_CHECK(!pin_memory.value_or(false), "Only dense CPU tensors can be pinned");
  const int dev = (device.has_value() && device->has_index()) ? device->index() : current_device();
  return empty_strided_b200(size, stride, dtype.value_or(at::get_default_dtype_as_scalartype()), dev);
}

// ----------------------------------------------------------------------- copies
static bool same_dense_layout(const at::Tensor& a, const at::Tensor& b) {
  return a.sizes() == b.sizes() && a.strides() == b.strides() && a.is_non_overlapping_and_dense();
}

static at::Tensor as_cpu_alias(const at::Tensor& t) {
  // Host simulation only: device memory is host memory.
  return at::from_blob(t.data_ptr(), t.sizes(), t.strides(),
                       at::TensorOptions().dtype(t.scalar_type()).device(at::kCPU));
}

// Device-to-device copy with arbitrary strides and dtypes on the current queue.
static void copy_d2d(const at::Tensor& src, const at::Tensor& dst, const OpScope& scope) {
  if (dst.numel() == 0) return;
  if (hostsim()) {
    as_cpu_alias(dst).copy_(as_cpu_alias(src.expand_as(dst)));
    return;
  }
  if (src.device() != dst.device()) {
    // Cross-device: stage through a dense tensor of dst's dtype on the source
    // device, move it with a peer copy, then scatter on the destination.
    at::Tensor s = src;
    if (s.scalar_type() != dst.scalar_type() || !s.is_contiguous() || s.sizes() != dst.sizes()) {
      at::Tensor tmp = empty_b200(dst.sizes(), dst.scalar_type(), src.device().index());
      OpScope sscope("copy_(staging)", src);
      launch_copy(s.expand_as(dst), tmp, sscope.stream());
      getCurrentQueue(src.device().index()).synchronize();
      s = tmp;
    } else {
      getCurrentQueue(src.device().index()).synchronize();
    }
    at::Tensor d = dst.is_contiguous() ? dst : empty_b200(dst.sizes(), dst.scalar_type(), dst.device().index());
    backend().memcpy_peer_async(d.data_ptr(), dst.device().index(), s.data_ptr(), src.device().index(), s.nbytes(),
                                scope.stream());
    if (!d.is_same(dst)) launch_copy(d, dst, scope.stream());
    scope.queue().synchronize();  // keeps `s` alive until the peer copy is done
    return;
  }
  if (src.scalar_type() == dst.scalar_type() && same_dense_layout(src, dst)) {
    backend().memcpy_async(dst.data_ptr(), src.data_ptr(), dst.nbytes(), CopyKind::D2D, scope.stream());
    return;
  }
  launch_copy(src.expand_as(dst), dst, scope.stream());
}

static at::Tensor b200_copy_from(const at::Tensor& self, const at::Tensor& dst, bool non_blocking);

// Lazy conjugate / negative views (x.conj(), the views autograd makes for complex gradients): the bits are metadata, the
// memory holds the unconjugated values.  The raw values are copied and the mathematical difference between source
// and destination is then applied to the destination in place.
static at::Tensor copy_with_lazy_bits(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
  at::Tensor src = self, out = dst;
  const bool flip_conj = src.is_conj() != out.is_conj(), flip_neg = src.is_neg() != out.is_neg();
  if (src.is_conj()) src = at::_conj(src);      // the same memory without the bit
  if (src.is_neg()) src = at::_neg_view(src);
  if (out.is_conj()) out = at::_conj(out);
  if (out.is_neg()) out = at::_neg_view(out);
  b200_copy_from(src, out, non_blocking);
  if (flip_conj && out.is_complex()) {
    if (is_b200(out)) at::view_as_real(out).select(-1, 1).neg_();  // conjugate in place: negate the imaginary parts
    else out.conj_physical_();
  }
  if (flip_neg) out.neg_();
  return dst;
}

static at::Tensor b200_copy_from(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
  TORCH_CHECK(self.defined() && dst.defined(), "copy_: undefined tensor");
  if (dst.numel() == 0) return dst;
  if (self.is_conj() || self.is_neg() || dst.is_conj() || dst.is_neg()) return copy_with_lazy_bits(self, dst, non_blocking);
  const bool src_dev = is_b200(self), dst_dev = is_b200(dst);
  if (src_dev && dst_dev) {
    OpScope scope("copy_(D2D)", dst);
    copy_d2d(self, dst, scope);
    return dst;
  }
  if (dst_dev) {  // host -> device
    TORCH_CHECK(self.device().is_cpu(), "b200 copy_: unsupported source device ", self.device());
    OpScope scope("copy_(H2D)", dst);
    at::Tensor src = self.expand_as(dst);
    if (dst.is_non_overlapping_and_dense()) {
      // Make the host tensor match dst's dtype and memory layout, then one DMA.
      at::Tensor host = src;
      const bool direct = src.scalar_type() == dst.scalar_type() && src.strides() == dst.strides() &&
                          src.sizes() == dst.sizes();
      if (!direct) {
        host = at::empty_strided(dst.sizes(), dst.strides(), src.options().dtype(dst.scalar_type()));
        host.copy_(src);
      }
      const bool pinned = isPinnedPtr(host.data_ptr());
      backend().memcpy_async(dst.data_ptr(), host.data_ptr(), dst.nbytes(), CopyKind::H2D, scope.stream());
      if (pinned) pinnedRecordQueue(host.data_ptr(), scope.queue());
      if (!(non_blocking && pinned && direct)) scope.queue().synchronize();
    } else {
      at::Tensor staged = empty_b200(dst.sizes(), dst.scalar_type(), dst.device().index());
      at::Tensor host = src.to(dst.scalar_type()).contiguous();
      backend().memcpy_async(staged.data_ptr(), host.data_ptr(), staged.nbytes(), CopyKind::H2D, scope.stream());
      scope.queue().synchronize();
      copy_d2d(staged, dst, scope);
    }
    return dst;
  }
  // device -> host
  TORCH_CHECK(src_dev && dst.device().is_cpu(), "b200 copy_: unsupported device pair ", self.device(), " -> ",
              dst.device());
  OpScope scope("copy_(D2H)", self);
  at::Tensor src = self.expand_as(dst);
  const bool direct = src.scalar_type() == dst.scalar_type() && src.strides() == dst.strides() &&
                      src.is_non_overlapping_and_dense();
  if (direct) {
    const bool pinned = isPinnedPtr(dst.data_ptr());
    backend().memcpy_async(dst.data_ptr(), src.data_ptr(), dst.nbytes(), CopyKind::D2H, scope.stream());
    if (pinned) pinnedRecordQueue(dst.data_ptr(), scope.queue());
    if (!(non_blocking && pinned)) scope.queue().synchronize();
    return dst;
  }
  // Make a dense device tensor with dst's dtype first (device-side cast), then DMA.
  at::Tensor dense = empty_b200(dst.sizes(), dst.scalar_type(), self.device().index());
  copy_d2d(src, dense, scope);
  if (dst.is_contiguous()) {
    backend().memcpy_async(dst.data_ptr(), dense.data_ptr(), dense.nbytes(), CopyKind::D2H, scope.stream());
    scope.queue().synchronize();
  } else {
    at::Tensor host = at::empty(dst.sizes(), dst.options());
    backend().memcpy_async(host.data_ptr(), dense.data_ptr(), dense.nbytes(), CopyKind::D2H, scope.stream());
    scope.queue().synchronize();
    dst.copy_(host);
  }
  return dst;
}

static at::Tensor b200_copy_from_and_resize(const at::Tensor& self, const at::Tensor& dst) {
  if (dst.sizes() != self.sizes()) dst.resize_(self.sizes());
  return b200_copy_from(self, dst, false);
}

static at::Scalar b200_local_scalar_dense(const at::Tensor& self) {
  TORCH_CHECK(self.numel() == 1, "a Tensor with ", self.numel(), " elements cannot be converted to Scalar");
  OpScope scope("_local_scalar_dense", self);
  alignas(16) char buf[16];
  backend().memcpy_async(buf, self.data_ptr(), self.element_size(), CopyKind::D2H, scope.stream());
  scope.queue().synchronize();
  at::Tensor host = at::from_blob(buf, {}, at::TensorOptions().dtype(self.scalar_type()).device(at::kCPU));
  return host.item();
}

// ------------------------------------------------------------------------ views
static at::Tensor& set_source_storage_offset(at::Tensor& result, at::Storage storage, int64_t storage_offset,
                                             c10::IntArrayRef size, c10::IntArrayRef stride) {
  at::native::checkSetStorage(result, std::move(storage), storage_offset, size, stride);
  c10::TensorImpl* impl = result.unsafeGetTensorImpl();
  impl->set_storage_offset(storage_offset);
  impl->set_sizes_and_strides(size, stride.data() ? stride : c10::IntArrayRef(at::infer_dense_strides(size, {})));
  // Grow the storage if the view would not fit.
  const size_t need = at::detail::computeStorageNbytes(impl->sizes(), impl->strides(), impl->dtype().itemsize(),
                                                       storage_offset);
  if (need > impl->storage().nbytes()) {
    at::detail::getPrivateUse1Hooks().resizePrivateUse1Bytes(impl->storage(), need);
  }
  return result;
}

static at::Tensor& set_source_storage(at::Tensor& result, at::Storage src) {
  const int64_t n = static_cast<int64_t>(src.nbytes() / result.dtype().itemsize());
  return set_source_storage_offset(result, std::move(src), 0, {n}, {1});
}

static at::Tensor& set_source_tensor(at::Tensor& result, const at::Tensor& src) {
  if (result.unsafeGetTensorImpl() != src.unsafeGetTensorImpl()) {
    set_source_storage_offset(result, src.storage(), src.storage_offset(), src.sizes(), src.strides());
  }
  return result;
}

static at::Tensor& set_empty(at::Tensor& result) {
  c10::Allocator* a = getB200CachingAllocator();
  auto st = c10::make_intrusive<c10::StorageImpl>(c10::StorageImpl::use_byte_size_t(), 0, a->allocate(0), a, true);
  return set_source_storage_offset(result, c10::Storage(std::move(st)), 0, {0}, {1});
}

static const at::Tensor& b200_resize_(const at::Tensor& self, c10::IntArrayRef size, std::optional<at::MemoryFormat> mf) {
  c10::TensorImpl* impl = self.unsafeGetTensorImpl();
  if (impl->sizes() == size && (!mf.has_value() || *mf == at::MemoryFormat::Contiguous ||
                                *mf == at::MemoryFormat::Preserve)) {
    return self;
  }
  impl->set_sizes_contiguous(size);
  if (mf.has_value() && *mf != at::MemoryFormat::Contiguous && *mf != at::MemoryFormat::Preserve) {
    impl->empty_tensor_restride(*mf);
  }
  const size_t need =
      at::detail::computeStorageNbytes(impl->sizes(), impl->strides(), impl->dtype().itemsize(), impl->storage_offset());
  if (need > impl->storage().nbytes()) {
    OpScope scope("resize_", self);
    at::detail::getPrivateUse1Hooks().resizePrivateUse1Bytes(impl->storage(), need);
  }
  return self;
}

static void b200_record_stream(at::Tensor& self, c10::Stream s) {
  recordQueue(self.storage().data_ptr(), Queue::from_c10(s));
}

// -------------------------------------------------------------------- pinning
static bool b200_is_pinned(const at::Tensor& self, std::optional<at::Device>) {
  return self.device().is_cpu() && isPinnedPtr(self.storage().data());
}
static at::Tensor b200_pin_memory(const at::Tensor& self, std::optional<at::Device>) {
  TORCH_CHECK(self.device().is_cpu(), "cannot pin '", self.toString(), "' only dense CPU tensors can be pinned");
  c10::Allocator* a = getB200PinnedAllocator();
  auto storage = c10::Storage(c10::Storage::use_byte_size_t(),
                              at::detail::computeStorageNbytes(self.sizes(), self.strides(), self.dtype().itemsize()),
                              a, /*resizable=*/false);
  at::Tensor out = at::empty({0}, self.options()).set_(storage, 0, self.sizes(), self.strides());
  out.copy_(self);
  return out;
}

TORCH_LIBRARY_IMPL(_, PrivateUse1, m) { m.fallback(torch::CppFunction::makeFromBoxedFunction<&cpu_fallback>()); }

// The generic kernels of the Conjugate / Negative keys materialise a lazy view by cloning it, and cloning ends in
// _copy_from again: these two operators handle the bits themselves (copy_with_lazy_bits), so the keys let them through.
TORCH_LIBRARY_IMPL(aten, Conjugate, m) {
  m.impl("_copy_from", torch::CppFunction::makeFallthrough());
  m.impl("_copy_from_and_resize", torch::CppFunction::makeFallthrough());
}
TORCH_LIBRARY_IMPL(aten, Negative, m) {
  m.impl("_copy_from", torch::CppFunction::makeFallthrough());
  m.impl("_copy_from_and_resize", torch::CppFunction::makeFallthrough());
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("empty.memory_format", TORCH_FN(empty_memory_format));
  m.impl("empty_strided", TORCH_FN(b200_empty_strided));
  m.impl("_copy_from", TORCH_FN(b200_copy_from));
  m.impl("_copy_from_and_resize", TORCH_FN(b200_copy_from_and_resize));
  m.impl("_local_scalar_dense", TORCH_FN(b200_local_scalar_dense));
  m.impl("as_strided", TORCH_FN(at::native::as_strided_tensorimpl));
  m.impl("view", TORCH_FN(at::native::view));
  m.impl("_reshape_alias", TORCH_FN(at::native::_reshape_alias));
  m.impl("unfold", TORCH_FN(at::native::unfold));
  // complex <-> real reinterpretation (rotary embeddings): pure metadata, and a view operator cannot go through the
  // CPU fallback (the result would be a copy, not a view)
  m.impl("view_as_real", TORCH_FN(at::native::view_as_real));
  m.impl("view_as_complex", TORCH_FN(at::native::view_as_complex));
  m.impl("set_.source_Storage_storage_offset", TORCH_FN(set_source_storage_offset));
  m.impl("set_.source_Storage", TORCH_FN(set_source_storage));
  m.impl("set_.source_Tensor", TORCH_FN(set_source_tensor));
  m.impl("set_", TORCH_FN(set_empty));
  m.impl("resize_", TORCH_FN(b200_resize_));
  m.impl("record_stream", TORCH_FN(b200_record_stream));
}

// Exposed to the Python layer (torch.b200.pin_memory / is_pinned).
at::Tensor pin_memory(const at::Tensor& t) { return b200_pin_memory(t, std::nullopt); }
bool tensor_is_pinned(const at::Tensor& t) { return b200_is_pinned(t, std::nullopt); }

}  // namespace ops
}  // namespace catch_b200
