#include "host_allocator.h"

#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <vector>

#include "device.h"
#include "log.h"
#include "notifier.h"

namespace catch_b200 {
namespace {

struct HostBlock {
  char* ptr = nullptr;
  size_t size = 0;
  bool in_use = false;
  std::vector<uint64_t> queues;  // queues that touched the block since it was handed out
};

struct BySize {
  bool operator()(const HostBlock* a, const HostBlock* b) const {
    return a->size != b->size ? a->size < b->size : a->ptr < b->ptr;
  }
};

class PinnedAllocator final : public c10::Allocator {
 public:
  c10::DataPtr allocate(size_t n) override {
    if (n == 0) return c10::DataPtr(nullptr, nullptr, &deleter, c10::Device(c10::DeviceType::CPU));
    std::lock_guard<std::mutex> g(mu_);
    drain();
    const size_t want = (n + 511) / 512 * 512;
    HostBlock key;
    key.size = want;
    HostBlock* b = nullptr;
    auto it = free_.lower_bound(&key);
    // Accept a cached block only if it wastes less than half of itself.
    if (it != free_.end() && (*it)->size <= 2 * want) {
      b = *it;
      free_.erase(it);
    } else {
      void* p = nullptr;
      int err = backend().try_host_alloc(&p, want);
      if (err != 0) {
        release_all_free();
        err = backend().try_host_alloc(&p, want);
      }
      TORCH_CHECK(err == 0, "b200: failed to allocate ", want, " bytes of pinned host memory (error ", err, ")");
      b = new HostBlock();
      b->ptr = static_cast<char*>(p);
      b->size = want;
      by_addr_[b->ptr] = b;
    }
    b->in_use = true;
    b->queues.clear();
    return c10::DataPtr(b->ptr, b->ptr, &deleter, c10::Device(c10::DeviceType::CPU));
  }
  c10::DeleterFnPtr raw_deleter() const override { return &deleter; }
  void copy_data(void* dest, const void* src, std::size_t count) const override { std::memcpy(dest, src, count); }

  void free_ptr(void* p) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = by_addr_.find(static_cast<char*>(p));
    if (it == by_addr_.end()) return;
    HostBlock* b = it->second;
    b->in_use = false;
    if (b->queues.empty()) {
      free_.insert(b);
      return;
    }
    Waiting w;
    w.block = b;
    for (uint64_t key : b->queues) {
      const int dev = static_cast<int>(key >> 32), id = static_cast<int>(key & 0xffffffffu);
      auto n = NotifierPool::instance().alloc(dev);
      n->place(getQueueById(dev, id));
      w.notifiers.emplace_back(std::move(n), dev);
    }
    b->queues.clear();
    waiting_.push_back(std::move(w));
  }

  HostBlock* find_containing(const void* p) {
    auto it = by_addr_.upper_bound(const_cast<char*>(static_cast<const char*>(p)));
    if (it == by_addr_.begin()) return nullptr;
    --it;
    HostBlock* b = it->second;
    const char* c = static_cast<const char*>(p);
    return (c >= b->ptr && c < b->ptr + b->size) ? b : nullptr;
  }

  bool is_pinned(const void* p) {
    std::lock_guard<std::mutex> g(mu_);
    HostBlock* b = find_containing(p);
    return b && b->in_use;
  }
  void record(const void* p, const Queue& q) {
    std::lock_guard<std::mutex> g(mu_);
    HostBlock* b = find_containing(p);
    if (!b) return;
    const uint64_t key = q.pack();
    for (uint64_t k : b->queues)
      if (k == key) return;
    b->queues.push_back(key);
  }
  void empty_cache() {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& w : waiting_)
      for (auto& n : w.notifiers) n.first->synchronize();
    drain();
    release_all_free();
  }
  size_t cached_bytes() {
    std::lock_guard<std::mutex> g(mu_);
    drain();  // blocks whose copies have finished count as cached
    size_t s = 0;
    for (auto* b : free_) s += b->size;
    return s;
  }
  static void deleter(void* p);

 private:
  struct Waiting {
    HostBlock* block;
    std::vector<std::pair<std::shared_ptr<Notifier>, int>> notifiers;
  };
  void drain() {
    for (auto it = waiting_.begin(); it != waiting_.end();) {
      bool done = true;
      for (auto& n : it->notifiers) done = done && n.first->query();
      if (done) {
        for (auto& n : it->notifiers) NotifierPool::instance().give_back(std::move(n.first), n.second);
        free_.insert(it->block);
        it = waiting_.erase(it);
      } else {
        ++it;
      }
    }
  }
  void release_all_free() {
    for (HostBlock* b : free_) {
      by_addr_.erase(b->ptr);
      backend().host_free(b->ptr);
      delete b;
    }
    free_.clear();
  }
  std::mutex mu_;
  std::set<HostBlock*, BySize> free_;
  std::map<char*, HostBlock*> by_addr_;
  std::deque<Waiting> waiting_;
};

PinnedAllocator& pinned() {
  static PinnedAllocator* a = new PinnedAllocator();
  return *a;
}
void PinnedAllocator::deleter(void* p) {
  try {
    pinned().free_ptr(p);
  } catch (const std::exception& e) {
    B200LOG(ERROR) << "b200 pinned allocator: exception while freeing: " << e.what();
  }
}

}  // namespace

c10::Allocator* getB200PinnedAllocator() { return &pinned(); }
bool isPinnedPtr(const void* p) { return pinned().is_pinned(p); }
void pinnedRecordQueue(const void* p, const Queue& q) { pinned().record(p, q); }
void pinnedEmptyCache() { pinned().empty_cache(); }
size_t pinnedCachedBytes() { return pinned().cached_bytes(); }

}  // namespace catch_b200
