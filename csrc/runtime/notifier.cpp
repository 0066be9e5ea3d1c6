#include "notifier.h"

#include "device.h"
#include "log.h"

namespace catch_b200 {

Notifier::~Notifier() { release(); }

void Notifier::release() {
  if (event_) {
    try {
      DeviceSwitch sw(device_);
      backend().event_destroy(event_);
    } catch (...) {
    }
    event_ = nullptr;
  }
}

void Notifier::move_from(Notifier&& o) {
  event_ = o.event_;
  device_ = o.device_;
  timing_ = o.timing_;
  placed_ = o.placed_;
  o.event_ = nullptr;
  o.placed_ = false;
}

void Notifier::create(int device) {
  DeviceSwitch sw(device);
  event_ = backend().event_create(timing_);
  device_ = device;
}

void Notifier::place() { place(getCurrentQueue()); }

void Notifier::place(const Queue& q) {
  if (!event_) create(q.device_index());
  TORCH_CHECK(device_ == q.device_index(), "Notifier device ", device_, " does not match placing queue's device ",
              q.device_index(), ".");
  DeviceSwitch sw(device_);
  backend().event_record(event_, q.handle());
  placed_ = true;
}

void Notifier::placeOnce(const Queue& q) {
  if (!placed_) place(q);
}

void Notifier::wait(const Queue& q) {
  if (!event_ || !placed_) return;  // nothing to wait for
  DeviceSwitch sw(q.device_index());
  backend().stream_wait_event(q.handle(), event_);
}

bool Notifier::query() const {
  if (!event_ || !placed_) return true;
  DeviceSwitch sw(device_);
  return backend().event_query(event_);
}

void Notifier::synchronize() const {
  if (!event_ || !placed_) return;
  DeviceSwitch sw(device_);
  backend().event_synchronize(event_);
}

float Notifier::elapsed_time(const Notifier& end) const {
  TORCH_CHECK(event_ && placed_ && end.event_ && end.placed_,
              "Both notifiers must be placed before calculating elapsed time.");
  TORCH_CHECK(timing_ && end.timing_, "Both notifiers must be created with timing enabled.");
  end.synchronize();
  DeviceSwitch sw(device_);
  return backend().event_elapsed_ms(event_, end.event_);
}

float Notifier::hardware_time(const Notifier& end) const { return elapsed_time(end) * 1000.0f; }

NotifierPool& NotifierPool::instance() {
  static NotifierPool* p = new NotifierPool();  // leaked: outlives static destruction order
  return *p;
}

std::shared_ptr<Notifier> NotifierPool::alloc(int device) {
  {
    std::lock_guard<std::mutex> g(mu_);
    auto& dq = pools_[device];
    if (!dq.empty()) {
      auto n = std::move(dq.front());
      dq.pop_front();
      return n;
    }
  }
  return std::make_shared<Notifier>(/*enable_timing=*/false);
}

void NotifierPool::give_back(std::shared_ptr<Notifier> n, int device) {
  std::lock_guard<std::mutex> g(mu_);
  pools_[device].push_back(std::move(n));
}

void NotifierPool::clean() {
  std::lock_guard<std::mutex> g(mu_);
  for (auto& dq : pools_) dq.clear();
}

size_t NotifierPool::cached(int device) {
  std::lock_guard<std::mutex> g(mu_);
  return pools_[device].size();
}

}  // namespace catch_b200
