// Notifier = a marker placed in a queue (a CUDA event on B200).
//
// Parity: torch_mlu/csrc/aten/device/notifier.h:37-83, notifier.cpp:36-112
// (lazy creation on the first placing queue's device, place / placeOnce /
// wait(queue) / query / synchronize / elapsed_time (ms) / hardware_time (us),
// move-only) and the per-device reuse pool of caching_notifier.h:16-42.
#pragma once
#include <deque>
#include <memory>
#include <mutex>
#include "queue.h"

namespace catch_b200 {

class Notifier {
 public:
  explicit Notifier(bool enable_timing = true) : timing_(enable_timing) {}
  ~Notifier();
  Notifier(const Notifier&) = delete;
  Notifier& operator=(const Notifier&) = delete;
  Notifier(Notifier&& o) noexcept { move_from(std::move(o)); }
  Notifier& operator=(Notifier&& o) noexcept {
    if (this != &o) {
      release();
      move_from(std::move(o));
    }
    return *this;
  }

  void place();                  // on the current queue
  void place(const Queue& q);
  void placeOnce(const Queue& q);  // no-op when already placed
  void wait(const Queue& q);     // q will not run later work until the marker is reached
  bool query() const;            // true if never placed or already reached
  void synchronize() const;      // host blocks
  float elapsed_time(const Notifier& end) const;   // milliseconds between the two markers
  float hardware_time(const Notifier& end) const;  // microseconds of device time between them
  bool is_created() const { return event_ != nullptr; }
  bool was_placed() const { return placed_; }
  int device_index() const { return device_; }
  void* handle() const { return event_; }

 private:
  void create(int device);
  void release();
  void move_from(Notifier&& o);
  void* event_ = nullptr;
  int device_ = -1;
  bool timing_ = true;
  bool placed_ = false;
};

// Pool of timing-disabled notifiers used by the allocators for deferred frees.
class NotifierPool {
 public:
  static NotifierPool& instance();
  std::shared_ptr<Notifier> alloc(int device);
  void give_back(std::shared_ptr<Notifier> n, int device);
  void clean();
  size_t cached(int device);

 private:
  std::mutex mu_;
  std::deque<std::shared_ptr<Notifier>> pools_[16];
};

}  // namespace catch_b200
