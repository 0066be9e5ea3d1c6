// Queue = an ordered stream of device work (a CUDA stream on B200).
//
// Parity: torch_mlu/csrc/aten/device/queue.h:68-196, queue.cpp:43-172 --
// a value type {handle, device, id}; one default queue per device; a pool of
// 32 queues per device handed out round-robin; a thread-local "current" queue
// per device; query / synchronize; a RAII guard (queue_guard.h:47-77).
// Differences on purpose: queues convert to and from c10::Stream so the device
// guard can exchange streams (the reference's exchangeStream is unimplemented,
// guard_impl.h:77-84), and the default queue is the CUDA default stream.
#pragma once
#include <c10/core/Stream.h>
#include <cstdint>
#include <functional>

namespace catch_b200 {

constexpr int kQueuesPerPool = 32;

class Queue {
 public:
  Queue() = default;
  Queue(void* handle, int device, int id) : handle_(handle), device_(device), id_(id) {}
  void* handle() const { return handle_; }
  int device_index() const { return device_; }
  int id() const { return id_; }  // 0 = default queue, 1..32 = pool slot
  bool is_default() const { return id_ == 0; }
  bool query() const;        // true when all submitted work has finished
  void synchronize() const;  // host blocks until the queue drains
  bool operator==(const Queue& o) const { return device_ == o.device_ && id_ == o.id_; }
  bool operator!=(const Queue& o) const { return !(*this == o); }
  uint64_t pack() const { return (static_cast<uint64_t>(device_) << 32) | static_cast<uint32_t>(id_); }
  c10::Stream to_c10() const;
  static Queue from_c10(const c10::Stream& s);

 private:
  void* handle_ = nullptr;
  int device_ = 0;
  int id_ = 0;
};

Queue getDefaultQueue(int device = -1);
Queue getCurrentQueue(int device = -1);
Queue getQueueFromPool(int device = -1);  // round-robin over the 32 pool queues
Queue getQueueById(int device, int id);
void setCurrentQueue(const Queue& q);
void synchronizeAllQueues(int device);

class QueueGuard {
 public:
  explicit QueueGuard(const Queue& q);
  ~QueueGuard();
  QueueGuard(const QueueGuard&) = delete;
  QueueGuard& operator=(const QueueGuard&) = delete;

 private:
  int prev_device_;
  Queue prev_queue_on_target_;
};

}  // namespace catch_b200

namespace std {
template <>
struct hash<catch_b200::Queue> {
  size_t operator()(const catch_b200::Queue& q) const noexcept { return std::hash<uint64_t>()(q.pack()); }
};
}  // namespace std
