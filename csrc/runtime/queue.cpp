#include "queue.h"

#include <array>
#include <atomic>
#include <mutex>

#include "device.h"
#include "log.h"

namespace catch_b200 {

namespace {
struct DeviceQueues {
  std::once_flag once;
  std::array<void*, kQueuesPerPool + 1> handles{};  // [0] = default (null handle on CUDA)
  std::atomic<uint32_t> next{0};
};
std::array<DeviceQueues, kMaxDevices> g_queues;

// Thread-local current queue id per device (0 = default).
int* tls_current() {
  thread_local int cur[kMaxDevices] = {0};
  return cur;
}

int resolve(int device) {
  if (device < 0) device = current_device();
  TORCH_CHECK(device < device_count() && device < kMaxDevices, "b200: invalid device ordinal ", device);
  return device;
}

DeviceQueues& ensure(int device) {
  DeviceQueues& dq = g_queues[device];
  std::call_once(dq.once, [&] {
    DeviceSwitch sw(device);
    // The default queue is the legacy default stream on CUDA (handle 0); the
    // host simulation needs a real object to hang the device index on.
    dq.handles[0] = hostsim() ? backend().stream_create(0) : nullptr;
    for (int i = 1; i <= kQueuesPerPool; ++i) dq.handles[i] = backend().stream_create(0);
  });
  return dq;
}
}  // namespace

bool Queue::query() const {
  DeviceSwitch sw(device_);
  return backend().stream_query(handle_);
}
void Queue::synchronize() const {
  DeviceSwitch sw(device_);
  backend().stream_synchronize(handle_);
}
c10::Stream Queue::to_c10() const {
  return c10::Stream(c10::Stream::UNSAFE, make_device(device_), static_cast<c10::StreamId>(id_));
}
Queue Queue::from_c10(const c10::Stream& s) {
  TORCH_CHECK(s.device_type() == c10::DeviceType::PrivateUse1, "b200: expected a b200 stream");
  return getQueueById(s.device_index(), static_cast<int>(s.id()));
}

Queue getQueueById(int device, int id) {
  device = resolve(device);
  TORCH_CHECK(id >= 0 && id <= kQueuesPerPool, "b200: invalid queue id ", id);
  return Queue(ensure(device).handles[id], device, id);
}
Queue getDefaultQueue(int device) { return getQueueById(resolve(device), 0); }
Queue getCurrentQueue(int device) {
  device = resolve(device);
  return getQueueById(device, tls_current()[device]);
}
Queue getQueueFromPool(int device) {
  device = resolve(device);
  DeviceQueues& dq = ensure(device);
  uint32_t n = dq.next.fetch_add(1, std::memory_order_relaxed);
  return getQueueById(device, 1 + static_cast<int>(n % kQueuesPerPool));
}
void setCurrentQueue(const Queue& q) {
  TORCH_CHECK(q.device_index() >= 0 && q.device_index() < kMaxDevices, "b200: bad queue device");
  tls_current()[q.device_index()] = q.id();
}
void synchronizeAllQueues(int device) {
  device = resolve(device);
  DeviceQueues& dq = ensure(device);
  DeviceSwitch sw(device);
  for (void* h : dq.handles) backend().stream_synchronize(h);
}

QueueGuard::QueueGuard(const Queue& q)
    : prev_device_(current_device()), prev_queue_on_target_(getCurrentQueue(q.device_index())) {
  if (q.device_index() != prev_device_) set_device(q.device_index());
  setCurrentQueue(q);
}
QueueGuard::~QueueGuard() {
  setCurrentQueue(prev_queue_on_target_);
  if (current_device() != prev_device_) backend().set_device(prev_device_);
}

}  // namespace catch_b200
