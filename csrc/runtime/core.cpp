// Registration of the b200 device with PyTorch's extension points:
// device guard, allocator, hooks, generator, tensor construction.
// Parity: guard_impl.h:43-89 + guard_impl.cpp:37 (guard), allocator.cpp:35-48
// (REGISTER_ALLOCATOR), generator_impl.cpp:72-271 (generator) of the reference
// -- all of which needed patches to PyTorch 1.6; here the PrivateUse1 extension
// points are used and PyTorch itself is untouched.
#include <ATen/EmptyTensor.h>
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <c10/core/impl/alloc_cpu.h>

#include "caching_allocator.h"
#include "device.h"
#include "generator.h"
#include "host_allocator.h"
#include "log.h"
#include "notifier.h"
#include "tensor_impl.h"

namespace catch_b200 {

// ------------------------------------------------------------------ TensorImpl
c10::intrusive_ptr<c10::TensorImpl> B200TensorImpl::shallow_copy_and_detach(const c10::VariableVersion& vc,
                                                                            bool allow) const {
  return detach_core(vc, allow);
}
c10::intrusive_ptr<c10::TensorImpl> B200TensorImpl::shallow_copy_and_detach(c10::VariableVersion&& vc,
                                                                            bool allow) const {
  return detach_core(std::move(vc), allow);
}
void B200TensorImpl::shallow_copy_from(const c10::intrusive_ptr<c10::TensorImpl>& impl) {
  c10::TensorImpl::shallow_copy_from(impl);
  if (auto* other = dynamic_cast<B200TensorImpl*>(impl.get())) channel_stats = other->channel_stats;
}

static at::Tensor make_b200_tensor(size_t nbytes, c10::ScalarType dtype, int device) {
  DeviceSwitch sw(device);
  c10::Allocator* a = getB200CachingAllocator();
  auto storage = c10::make_intrusive<c10::StorageImpl>(c10::StorageImpl::use_byte_size_t(), nbytes, a->allocate(nbytes),
                                                       a, /*resizable=*/true);
  constexpr c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  return at::detail::make_tensor<B200TensorImpl>(c10::Storage(std::move(storage)), ks,
                                                 c10::scalarTypeToTypeMeta(dtype));
}

at::Tensor empty_b200(c10::IntArrayRef size, c10::ScalarType dtype, int device, std::optional<c10::MemoryFormat> mf) {
  if (device < 0) device = current_device();
  at::detail::check_size_nonnegative(size);
  const size_t nbytes = at::detail::computeStorageNbytesContiguous(size, c10::elementSize(dtype));
  at::Tensor t = make_b200_tensor(nbytes, dtype, device);
  if (size.size() != 1 || size[0] != 0) t.unsafeGetTensorImpl()->set_sizes_contiguous(size);
  if (mf.has_value() && *mf != c10::MemoryFormat::Contiguous && *mf != c10::MemoryFormat::Preserve) {
    t.unsafeGetTensorImpl()->empty_tensor_restride(*mf);
  }
  return t;
}

at::Tensor empty_strided_b200(c10::IntArrayRef size, c10::IntArrayRef stride, c10::ScalarType dtype, int device) {
  if (device < 0) device = current_device();
  at::detail::check_size_nonnegative(size);
  const size_t nbytes = at::detail::computeStorageNbytes(size, stride, c10::elementSize(dtype));
  at::Tensor t = make_b200_tensor(nbytes, dtype, device);
  t.unsafeGetTensorImpl()->set_sizes_and_strides(size, stride);
  return t;
}

// ------------------------------------------------------------------- Generator
B200GeneratorImpl::B200GeneratorImpl(c10::DeviceIndex idx)
    : c10::GeneratorImpl(c10::Device(c10::DeviceType::PrivateUse1, idx),
                         c10::DispatchKeySet(c10::DispatchKey::PrivateUse1)) {}
void B200GeneratorImpl::set_current_seed(uint64_t seed) {
  seed_ = seed;
  offset_ = 0;
}
void B200GeneratorImpl::set_offset(uint64_t offset) { offset_ = offset; }
uint64_t B200GeneratorImpl::get_offset() const { return offset_; }
uint64_t B200GeneratorImpl::current_seed() const { return seed_; }
uint64_t B200GeneratorImpl::seed() {
  uint64_t s = c10::detail::getNonDeterministicRandom(false);
  set_current_seed(s);
  return s;
}
void B200GeneratorImpl::set_state(const c10::TensorImpl& new_state) {
  TORCH_CHECK(new_state.numel() == 16 && new_state.dtype() == caffe2::TypeMeta::Make<uint8_t>(),
              "b200 RNG state must be a 16-byte ByteTensor (seed, offset)");
  const uint8_t* p = static_cast<const uint8_t*>(new_state.data());
  std::memcpy(&seed_, p, 8);
  std::memcpy(&offset_, p + 8, 8);
}
c10::intrusive_ptr<c10::TensorImpl> B200GeneratorImpl::get_state() const {
  at::Tensor t = at::empty({16}, at::TensorOptions().dtype(at::kByte).device(at::kCPU));
  uint8_t* p = t.data_ptr<uint8_t>();
  std::memcpy(p, &seed_, 8);
  std::memcpy(p + 8, &offset_, 8);
  return t.getIntrusivePtr();
}
std::pair<uint64_t, uint64_t> B200GeneratorImpl::philox_engine_inputs(uint64_t increment) {
  // Offsets advance in multiples of 4 because one Philox call yields 4 words.
  increment = (increment + 3) / 4 * 4;
  uint64_t off = offset_;
  offset_ += increment;
  return {seed_, off};
}
B200GeneratorImpl* B200GeneratorImpl::clone_impl() const {
  auto* g = new B200GeneratorImpl(device_.index());
  g->seed_ = seed_;
  g->offset_ = offset_;
  return g;
}

const at::Generator& getDefaultB200Generator(c10::DeviceIndex device) {
  static std::vector<at::Generator> gens;
  static std::once_flag once;
  std::call_once(once, [] {
    const int n = std::max(device_count(), 1);
    gens.resize(n);
    for (int i = 0; i < n; ++i) gens[i] = at::make_generator<B200GeneratorImpl>(static_cast<c10::DeviceIndex>(i));
  });
  if (device < 0) device = static_cast<c10::DeviceIndex>(current_device());
  TORCH_CHECK(device < static_cast<int>(gens.size()), "b200: invalid device for generator: ", static_cast<int>(device));
  return gens[device];
}
at::Generator createB200Generator(c10::DeviceIndex device) {
  if (device < 0) device = static_cast<c10::DeviceIndex>(current_device());
  return at::make_generator<B200GeneratorImpl>(device);
}
void manual_seed(int device, uint64_t seed) {
  auto gen = getDefaultB200Generator(static_cast<c10::DeviceIndex>(device));
  std::lock_guard<std::mutex> lock(gen.mutex());
  gen.set_current_seed(seed);
}
void manual_seed_all(uint64_t seed) {
  for (int i = 0; i < device_count(); ++i) manual_seed(i, seed);
}

// ---------------------------------------------------------------- device guard
namespace {

struct B200GuardImpl final : public c10::impl::DeviceGuardImplInterface {
  static constexpr c10::DeviceType static_type = c10::DeviceType::PrivateUse1;
  B200GuardImpl() = default;
  explicit B200GuardImpl(c10::DeviceType t) { TORCH_INTERNAL_ASSERT(t == static_type); }

  c10::DeviceType type() const override { return static_type; }
  c10::Device exchangeDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.type() == static_type);
    c10::Device old = getDevice();
    if (old.index() != d.index()) set_device(d.index());
    return old;
  }
  c10::Device getDevice() const override { return make_device(current_device()); }
  void setDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.type() == static_type);
    if (current_device() != d.index()) set_device(d.index());
  }
  void uncheckedSetDevice(c10::Device d) const noexcept override {
    try {
      backend().set_device(d.index());
    } catch (...) {
    }
  }
  c10::Stream getStream(c10::Device d) const noexcept override { return getCurrentQueue(d.index()).to_c10(); }
  c10::Stream getDefaultStream(c10::Device d) const override { return getDefaultQueue(d.index()).to_c10(); }
  c10::Stream getStreamFromGlobalPool(c10::Device d, bool) const override {
    return getQueueFromPool(d.index()).to_c10();
  }
  c10::Stream getNewStream(c10::Device d, int) const override { return getQueueFromPool(d.index()).to_c10(); }
  c10::Stream exchangeStream(c10::Stream s) const noexcept override {
    Queue q = Queue::from_c10(s);
    c10::Stream old = getCurrentQueue(q.device_index()).to_c10();
    setCurrentQueue(q);
    return old;
  }
  void* getStreamNativeHandle(const c10::Stream s) const override { return Queue::from_c10(s).handle(); }
  c10::DeviceIndex deviceCount() const noexcept override {
    try {
      return static_cast<c10::DeviceIndex>(device_count());
    } catch (...) {
      return 0;
    }
  }

  // Events are Notifier objects owned through the void* slot.
  void destroyEvent(void* event, const c10::DeviceIndex) const noexcept override {
    delete static_cast<Notifier*>(event);
  }
  void record(void** event, const c10::Stream& stream, const c10::DeviceIndex device_index,
              const c10::EventFlag flag) const override {
    TORCH_CHECK(device_index == -1 || device_index == stream.device_index(), "Event device index ", device_index,
                " does not match recording stream's device index ", stream.device_index(), ".");
    if (!*event) *event = new Notifier(flag == c10::EventFlag::BACKEND_DEFAULT ? true : false);
    static_cast<Notifier*>(*event)->place(Queue::from_c10(stream));
  }
  void block(void* event, const c10::Stream& stream) const override {
    if (!event) return;
    static_cast<Notifier*>(event)->wait(Queue::from_c10(stream));
  }
  bool queryEvent(void* event) const override { return !event || static_cast<Notifier*>(event)->query(); }
  bool queryStream(const c10::Stream& s) const override { return Queue::from_c10(s).query(); }
  void synchronizeStream(const c10::Stream& s) const override { Queue::from_c10(s).synchronize(); }
  void synchronizeEvent(void* event) const override {
    if (event) static_cast<Notifier*>(event)->synchronize();
  }
  void synchronizeDevice(const c10::DeviceIndex d) const override { synchronize(d); }
  void recordDataPtrOnStream(const c10::DataPtr& p, const c10::Stream& s) const override {
    recordQueue(p, Queue::from_c10(s));
  }
  double elapsedTime(void* e1, void* e2, const c10::DeviceIndex) const override {
    TORCH_CHECK(e1 && e2, "Both events must be recorded before calculating elapsed time.");
    return static_cast<Notifier*>(e1)->elapsed_time(*static_cast<Notifier*>(e2));
  }
};

C10_REGISTER_GUARD_IMPL(PrivateUse1, B200GuardImpl);

// ------------------------------------------------------------------------ hooks
struct B200Hooks final : public at::PrivateUse1HooksInterface {
  bool isBuilt() const override { return true; }
  bool isAvailable() const override { return device_count() > 0; }
  const at::Generator& getDefaultGenerator(c10::DeviceIndex idx) const override { return getDefaultB200Generator(idx); }
  at::Generator getNewGenerator(c10::DeviceIndex idx) const override { return createB200Generator(idx); }
  at::Device getDeviceFromPtr(void*) const override { return make_device(current_device()); }
  bool isPinnedPtr(const void* data) const override { return catch_b200::isPinnedPtr(data); }
  at::Allocator* getPinnedMemoryAllocator() const override { return getB200PinnedAllocator(); }
  bool hasPrimaryContext(c10::DeviceIndex) const override { return true; }
  c10::DeviceIndex deviceCount() const override { return static_cast<c10::DeviceIndex>(device_count()); }
  void setCurrentDevice(c10::DeviceIndex d) const override { set_device(d); }
  c10::DeviceIndex getCurrentDevice() const override { return static_cast<c10::DeviceIndex>(current_device()); }
  c10::DeviceIndex exchangeDevice(c10::DeviceIndex d) const override {
    auto old = static_cast<c10::DeviceIndex>(current_device());
    if (d != old) set_device(d);
    return old;
  }
  c10::DeviceIndex maybeExchangeDevice(c10::DeviceIndex d) const override { return exchangeDevice(d); }
  void resizePrivateUse1Bytes(const c10::Storage& storage, size_t newsize) const override {
    c10::StorageImpl* st = storage.unsafeGetStorageImpl();
    TORCH_CHECK(st->resizable(), "Trying to resize storage that is not resizable");
    const size_t old = st->nbytes();
    if (newsize == old) return;
    const int device = st->device().index();
    DeviceSwitch sw(device);
    c10::DataPtr fresh = newsize ? getB200CachingAllocator()->allocate(newsize)
                                 : c10::DataPtr(nullptr, nullptr, getB200CachingAllocator()->raw_deleter(),
                                                make_device(device));
    if (old && newsize && st->data()) {
      backend().memcpy_async(fresh.get(), st->data(), std::min(old, newsize), CopyKind::D2D,
                             getCurrentQueue(device).handle());
    }
    st->set_data_ptr_noswap(std::move(fresh));
    st->set_nbytes(newsize);
  }
};

struct Registrar {
  Registrar() {
    c10::SetAllocator(c10::DeviceType::PrivateUse1, getB200CachingAllocator());
    at::RegisterPrivateUse1HooksInterface(new B200Hooks());
  }
};
static Registrar g_registrar;

}  // namespace
}  // namespace catch_b200
