#include "device.h"

#include <array>
#include <mutex>
#include <sstream>

#include "log.h"

namespace catch_b200 {

int device_count() { return backend().device_count(); }

void check_versions_once() {
  static std::once_flag once;
  std::call_once(once, [] {
    if (hostsim()) return;
    int rt = 0, drv = 0;
    backend().versions(&rt, &drv);
    // Built against CUDA 12.x; sm_100a code needs a driver that knows CUDA >= 12.8.
    constexpr int kMinDriver = 12080;
    if (drv < kMinDriver) {
      B200LOG(WARNING) << "CUDA driver API version " << drv << " is older than the required " << kMinDriver
                       << "; sm_100a kernels may fail to load.";
    }
    const DeviceProp p = backend().device_props(backend().get_device());
    if (p.major != 10) {
      B200LOG(WARNING) << "device '" << p.name << "' has compute capability " << p.major << "." << p.minor
                       << "; this backend ships sm_100a code only.";
    }
  });
}

void set_device(int device) {
  TORCH_CHECK(device >= 0 && device < device_count(), "b200: invalid device ordinal ", device, " (device count ",
              device_count(), ")");
  backend().set_device(device);
  check_versions_once();
}

int current_device() { return backend().get_device(); }

DeviceSwitch::DeviceSwitch(int device) : prev_(backend().get_device()), changed_(false) {
  if (device >= 0 && device != prev_) {
    backend().set_device(device);
    changed_ = true;
  }
}
DeviceSwitch::~DeviceSwitch() {
  if (changed_) backend().set_device(prev_);
}

void synchronize(int device) {
  DeviceSwitch sw(device);
  backend().device_synchronize();
}

const DeviceProp& device_properties(int device) {
  static std::array<DeviceProp, kMaxDevices> props;
  static std::array<std::once_flag, kMaxDevices> flags_;
  TORCH_CHECK(device >= 0 && device < device_count() && device < kMaxDevices, "b200: invalid device ordinal ", device);
  std::call_once(flags_[device], [&] { props[device] = backend().device_props(device); });
  return props[device];
}

std::string version_string() {
  std::ostringstream os;
  int rt = 0, drv = 0;
  backend().versions(&rt, &drv);
  os << "catch_b200 0.1.0 (backend=" << backend().name() << ", cuda_runtime=" << rt << ", cuda_driver=" << drv << ")";
  return os.str();
}

}  // namespace catch_b200
