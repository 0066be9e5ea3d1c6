// Device management for the b200 backend.
// Parity: torch_mlu/csrc/aten/device/device.h:39-84, device.cpp:67-121
// (device_count / setDevice with one-time version check / current_device /
// synchronize / lazily initialised per-device properties).
#pragma once
#include <c10/core/Device.h>
#include <cstddef>
#include "backend.h"

namespace catch_b200 {

constexpr int kMaxDevices = 16;

int device_count();
void set_device(int device);     // first call also runs the one-time version check
int current_device();
void synchronize(int device = -1);
const DeviceProp& device_properties(int device);
// Runs fn-style code with `device` current and restores the previous device.
struct DeviceSwitch {
  explicit DeviceSwitch(int device);
  ~DeviceSwitch();
  int prev_;
  bool changed_;
};
inline c10::Device make_device(int idx) {
  return c10::Device(c10::DeviceType::PrivateUse1, static_cast<c10::DeviceIndex>(idx));
}
void hostsim_set_memory_limit(size_t bytes);

// Version report: library versions seen at run time vs the ones required at
// build time (parity: torch_mlu/tools/template/version.cpp:36-139).
std::string version_string();
void check_versions_once();

}  // namespace catch_b200
