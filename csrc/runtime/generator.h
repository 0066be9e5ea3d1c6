// Philox counter-based random generator state for the b200 device.
// Parity: torch_mlu/csrc/aten/core/generator_impl.h:38-67 (per-device default
// generator, manual_seed / manual_seed_all, create).  The reference keeps an
// MTGP32 state tensor on the device; Philox needs only (seed, offset) on the host.
#pragma once
#include <ATen/core/Generator.h>
#include <c10/core/GeneratorImpl.h>
#include <utility>

namespace catch_b200 {

class B200GeneratorImpl final : public c10::GeneratorImpl {
 public:
  explicit B200GeneratorImpl(c10::DeviceIndex device_index = -1);
  void set_current_seed(uint64_t seed) override;
  void set_offset(uint64_t offset) override;
  uint64_t get_offset() const override;
  uint64_t current_seed() const override;
  uint64_t seed() override;
  void set_state(const c10::TensorImpl& new_state) override;
  c10::intrusive_ptr<c10::TensorImpl> get_state() const override;
  // Reserve `increment` Philox counters (each yields 4 x 32 random bits per
  // thread) and return the (seed, offset) pair a kernel should start from.
  std::pair<uint64_t, uint64_t> philox_engine_inputs(uint64_t increment);
  static c10::DeviceType device_type() { return c10::DeviceType::PrivateUse1; }

 private:
  B200GeneratorImpl* clone_impl() const override;
  uint64_t seed_ = 67280421310721ULL;  // same default seed as the stock generators
  uint64_t offset_ = 0;
};

const at::Generator& getDefaultB200Generator(c10::DeviceIndex device = -1);
at::Generator createB200Generator(c10::DeviceIndex device = -1);
void manual_seed(int device, uint64_t seed);
void manual_seed_all(uint64_t seed);

}  // namespace catch_b200
