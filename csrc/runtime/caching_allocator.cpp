#include "caching_allocator.h"

#include <functional>

#include <c10/core/CPUAllocator.h>
#include <c10/util/Exception.h>
#include <c10/util/Type.h>
#include <execinfo.h>
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <vector>
#include <array>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <set>
#include <sstream>
#include <unordered_map>
#include <unordered_set>

#include "device.h"
#include "log.h"
#include "notifier.h"

namespace catch_b200 {

namespace {

constexpr size_t kRound = 512;                 // every block size is a multiple of this
constexpr size_t kSmallLimit = 1 << 20;        // requests up to 1 MiB use the small pool
constexpr size_t kSmallSegment = 2 << 20;      // small pool grows in 2 MiB segments
constexpr size_t kMidLimit = 10 << 20;         // requests below this get a 20 MiB segment
constexpr size_t kMidSegment = 20 << 20;
constexpr size_t kLargeRound = 2 << 20;        // bigger segments are rounded to 2 MiB
constexpr size_t kGuard = 512;                 // debug guard region on each side
constexpr uint8_t kGuardByte = 0xA5;
thread_local uint64_t t_private_pool = 0;  // pool that this thread's allocations use (graph capture)
std::atomic<AllocationContextHook> g_context_hook{nullptr};

inline size_t round_up(size_t n, size_t m) { return (n + m - 1) / m * m; }

struct Block {
  int device = 0;
  uint64_t queue_key = 0;  // Queue::pack() of the allocating queue
  size_t size = 0;         // bytes of this block (guards included in debug mode)
  char* ptr = nullptr;
  bool small = false;
  bool in_use = false;
  Block* prev = nullptr;   // neighbours inside the same segment
  Block* next = nullptr;
  int pending_events = 0;  // outstanding cross-queue notifiers
  std::unordered_set<uint64_t> other_queues;  // queues recorded through recordQueue
  size_t requested = 0;    // user-visible size (debug report)
  // debug mode: where the block was handed out (native return addresses, context text of the hook)
  std::vector<void*> origin_frames;
  std::string origin_context;
  // 0 = the shared cache; otherwise the private pool of a captured graph: its free blocks serve only
  // allocations made while that graph is being captured, so memory whose address is baked into the graph is
  // never handed to anybody else while the graph exists
  uint64_t pool = 0;
  bool guarded = false;    // handed out in debug mode: guard regions on both sides of the user range
};

struct BlockLess {
  bool operator()(const Block* a, const Block* b) const {
    if (a->pool != b->pool) return a->pool < b->pool;
    if (a->queue_key != b->queue_key) return a->queue_key < b->queue_key;
    if (a->size != b->size) return a->size < b->size;
    return a->ptr < b->ptr;
  }
};
using Pool = std::set<Block*, BlockLess>;

struct PendingFree {
  std::shared_ptr<Notifier> n;
  Block* block;
};

struct DeviceState {
  Pool small_free, large_free;
  MemoryStats stats;
  std::deque<PendingFree> pending;
  int64_t reserve_limit = 0;  // > 0: the allocator may not hold more than this many bytes of device memory
};

class CachingAllocator final : public c10::Allocator {
 public:
  CachingAllocator() { debug_ = flags().memory_debug; }

  // ---------------------------------------------------------------- allocate
  void* malloc_block(size_t bytes, int device, const Queue& q) {
    // The context hook may take the interpreter lock: it runs before this allocator's own lock is taken, so a
    // thread that holds the interpreter lock and waits for the allocator cannot deadlock with this one.
    std::string context;
    if (debug_) {
      if (AllocationContextHook hook = g_context_hook.load()) context = hook();
    }
    std::lock_guard<std::recursive_mutex> g(mu_);
    DeviceState& st = state(device);
    drain_pending(st);
    const size_t want = round_up(std::max<size_t>(bytes, 1), kRound) + (debug_ ? 2 * kGuard : 0);
    const bool small = want <= kSmallLimit;
    Pool& pool = small ? st.small_free : st.large_free;

    Block key;
    key.queue_key = q.pack();
    key.size = want;
    key.ptr = nullptr;
    key.pool = t_private_pool;
    Block* blk = nullptr;
    auto it = pool.lower_bound(&key);
    if (it != pool.end() && (*it)->queue_key == key.queue_key && (*it)->pool == key.pool) {
      blk = *it;
      pool.erase(it);
    } else {
      blk = grow(st, device, q, want, small);
    }
    // Split when the remainder is worth keeping.
    const size_t remain = blk->size - want;
    const bool split = small ? remain >= kRound : remain > kSmallLimit;
    if (split) {
      Block* rest = new Block();
      rest->device = device;
      rest->queue_key = blk->queue_key;
      rest->pool = blk->pool;
      rest->size = remain;
      rest->ptr = blk->ptr + want;
      rest->small = small;
      rest->prev = blk;
      rest->next = blk->next;
      if (rest->next) rest->next->prev = rest;
      blk->next = rest;
      blk->size = want;
      pool.insert(rest);
    }
    blk->in_use = true;
    blk->requested = bytes;
    st.stats.allocated += static_cast<int64_t>(blk->size);
    st.stats.max_allocated = std::max(st.stats.max_allocated, st.stats.allocated);
    st.stats.num_alloc++;
    blk->guarded = debug_;
    char* user = blk->ptr + (debug_ ? kGuard : 0);
    if (debug_) {
      paint_guards(blk, q);
      record_origin(blk, std::move(context));
    }
    live_[user] = blk;
    c10::reportMemoryUsageToProfiler(user, static_cast<int64_t>(blk->size), st.stats.allocated, st.stats.reserved,
                                     make_device(device));
    return user;
  }

  // -------------------------------------------------------------------- free
  void free_block(void* user) {
    if (!user) return;
    std::lock_guard<std::recursive_mutex> g(mu_);
    auto it = live_.find(user);
    TORCH_CHECK(it != live_.end(), "b200 allocator: freeing a pointer it does not own: ", user);
    Block* blk = it->second;
    live_.erase(it);
    DeviceState& st = state(blk->device);
    if (blk->guarded) {
      std::string why;
      if (!verify_guards(blk, &why)) {
        B200LOG(ERROR) << "memory debug: out-of-bounds write detected on free: " << why;
        corrupted_on_free_++;
        last_corruption_ = why;
      }
    }
    blk->in_use = false;
    blk->guarded = false;
    blk->origin_frames.clear();
    blk->origin_context.clear();
    st.stats.allocated -= static_cast<int64_t>(blk->size);
    st.stats.num_free++;
    c10::reportMemoryUsageToProfiler(user, -static_cast<int64_t>(blk->size), st.stats.allocated, st.stats.reserved,
                                     make_device(blk->device));
    if (!blk->other_queues.empty() && t_private_pool != 0) blk->other_queues.clear();  // no notifiers inside a capture
    if (!blk->other_queues.empty()) {
      // The block was also used on other queues: give it back only after
      // everything those queues have been asked to do so far has finished.
      std::unordered_set<uint64_t> qs;
      qs.swap(blk->other_queues);
      for (uint64_t key : qs) {
        const int dev = static_cast<int>(key >> 32);
        const int id = static_cast<int>(key & 0xffffffffu);
        auto n = NotifierPool::instance().alloc(dev);
        n->place(getQueueById(dev, id));
        blk->pending_events++;
        state(dev).pending.push_back({std::move(n), blk});
      }
      return;
    }
    release_to_pool(blk);
  }

  void record_queue(void* user, const Queue& q) {
    if (!user) return;
    std::lock_guard<std::recursive_mutex> g(mu_);
    auto it = live_.find(user);
    if (it == live_.end()) return;  // not ours (e.g. an empty tensor)
    Block* blk = it->second;
    if (q.pack() == blk->queue_key) return;
    blk->other_queues.insert(q.pack());
  }

  void empty_cache() {
    std::lock_guard<std::recursive_mutex> g(mu_);
    for (int d = 0; d < kMaxDevices; ++d) {
      if (!states_[d]) continue;
      DeviceState& st = *states_[d];
      sync_pending(st);
      release_segments(st, st.small_free, d);
      release_segments(st, st.large_free, d);
    }
  }

  MemoryStats stats(int device) {
    std::lock_guard<std::recursive_mutex> g(mu_);
    return state(device).stats;
  }
  void reset_peak(int device) {
    std::lock_guard<std::recursive_mutex> g(mu_);
    MemoryStats& s = state(device).stats;
    s.max_allocated = s.allocated;
    s.max_reserved = s.reserved;
  }

  // ------------------------------------------------------- graph-private pools
  uint64_t new_pool() {
    std::lock_guard<std::recursive_mutex> g(mu_);
    return ++next_pool_;
  }
  // The graph that owned `pool` was destroyed: its free blocks join the shared cache now, blocks still in use
  // (tensors the capture returned) follow when they are freed.
  void retire_pool(uint64_t pool) {
    if (pool == 0) return;
    std::lock_guard<std::recursive_mutex> g(mu_);
    retired_pools_.insert(pool);
    for (int d = 0; d < kMaxDevices; ++d) {
      if (!states_[d]) continue;
      for (Pool* fp : {&states_[d]->small_free, &states_[d]->large_free}) {
        std::vector<Block*> mine;
        for (Block* b : *fp)
          if (b->pool == pool) mine.push_back(b);
        // free neighbours were merged when they were freed, so relabelling is all that is needed
        for (Block* b : mine) {
          fp->erase(b);
          b->pool = 0;
          fp->insert(b);
        }
      }
    }
  }

  void set_native(bool v) { native_ = v; }
  void set_reserve_limit(int device, int64_t bytes) {
    std::lock_guard<std::recursive_mutex> g(mu_);
    state(device).reserve_limit = bytes;
  }
  int64_t reserve_limit(int device) {
    std::lock_guard<std::recursive_mutex> g(mu_);
    return state(device).reserve_limit;
  }
  bool native() const { return native_; }
  // Blocks handed out before the switch keep their layout (each block remembers whether it has guards), so the
  // mode can change while tensors are alive; only blocks allocated in debug mode are checked.
  void set_debug(bool v) {
    std::lock_guard<std::recursive_mutex> g(mu_);
    debug_ = v;
  }
  bool debug() const { return debug_; }

  DebugReport debug_check(const void* user) {
    std::lock_guard<std::recursive_mutex> g(mu_);
    DebugReport r;
    r.corrupted = corrupted_on_free_;
    if (corrupted_on_free_) r.detail = "(freed) " + last_corruption_ + "\n";
    if (!debug_) return r;
    auto check = [&](Block* b) {
      if (!b->guarded) return;
      r.blocks_checked++;
      std::string why;
      if (!verify_guards(b, &why)) {
        r.corrupted++;
        r.detail += why + "\n";
      }
    };
    if (user) {
      auto it = live_.find(const_cast<void*>(user));
      TORCH_CHECK(it != live_.end(), "memory_debug: pointer is not a live b200 block");
      check(it->second);
    } else {
      for (auto& kv : live_) check(kv.second);
    }
    return r;
  }

  std::string origin_of(const void* user) {
    std::lock_guard<std::recursive_mutex> g(mu_);
    auto it = live_.find(const_cast<void*>(user));
    return it == live_.end() ? std::string() : format_origin(it->second);
  }

  std::string summary(int device) {
    MemoryStats s = stats(device);
    std::ostringstream os;
    os << "b200:" << device << " allocated " << s.allocated << " B (peak " << s.max_allocated << " B), reserved "
       << s.reserved << " B (peak " << s.max_reserved << " B), segments " << s.num_segments << ", allocs "
       << s.num_alloc << ", frees " << s.num_free << ", OOMs " << s.num_ooms << ", retries " << s.num_retries;
    return os.str();
  }

  // -------------------------------------------------- c10::Allocator interface
  c10::DataPtr allocate(size_t n) override {
    const int device = current_device();
    if (n == 0) return c10::DataPtr(nullptr, nullptr, &deleter, make_device(device));
    void* p = malloc_block(n, device, getCurrentQueue(device));
    return c10::DataPtr(p, p, &deleter, make_device(device));
  }
  c10::DeleterFnPtr raw_deleter() const override { return &deleter; }
  void copy_data(void* dest, const void* src, std::size_t count) const override {
    Queue q = getCurrentQueue();
    backend().memcpy_async(dest, src, count, CopyKind::D2D, q.handle());
  }
  static void deleter(void* p);

 private:
  DeviceState& state(int device) {
    TORCH_CHECK(device >= 0 && device < kMaxDevices, "b200 allocator: bad device ", device);
    if (!states_[device]) states_[device] = std::make_unique<DeviceState>();
    return *states_[device];
  }

  size_t segment_size(size_t want, bool small, int device) {
    if (small) return kSmallSegment;
    if (native_) return round_up(want, kRound);
    if (want < kMidLimit) return kMidSegment;
    (void)device;
    return round_up(want, kLargeRound);
  }

  Block* grow(DeviceState& st, int device, const Queue& q, size_t want, bool small) {
    const size_t seg = segment_size(want, small, device);
    DeviceSwitch sw(device);
    void* p = nullptr;
    // a per-process limit (set_per_process_memory_fraction) is treated like an allocation failure of the driver
    auto over_limit = [&] { return st.reserve_limit > 0 && st.stats.reserved + static_cast<int64_t>(seg) > st.reserve_limit; };
    int err = over_limit() ? -1 : backend().try_malloc(&p, seg);
    if (err != 0) {
      // Give cached memory back to the driver and try again.
      st.stats.num_retries++;
      sync_pending(st);
      release_segments(st, st.small_free, device);
      release_segments(st, st.large_free, device);
      err = over_limit() ? -1 : backend().try_malloc(&p, seg);
    }
    if (err != 0) {
      st.stats.num_ooms++;
      size_t free_b = 0, total_b = 0;
      try {
        backend().mem_info(&free_b, &total_b);
      } catch (...) {
      }
      TORCH_CHECK_WITH(OutOfMemoryError, false, "b200 out of memory. Tried to allocate ", seg, " bytes for a request of ",
                       want, " bytes (device ", device, "; ", total_b, " bytes total capacity; ", free_b,
                       " bytes free; ", st.stats.allocated, " bytes already allocated; ", st.stats.reserved,
                       " bytes reserved by the caching allocator",
                       st.reserve_limit > 0 ? "; per-process limit " + std::to_string(st.reserve_limit) + " bytes" : std::string(), ").");
    }
    Block* b = new Block();
    b->device = device;
    b->queue_key = q.pack();
    b->pool = t_private_pool;
    b->size = seg;
    b->ptr = static_cast<char*>(p);
    b->small = small;
    st.stats.reserved += static_cast<int64_t>(seg);
    st.stats.max_reserved = std::max(st.stats.max_reserved, st.stats.reserved);
    st.stats.num_segments++;
    return b;
  }

  void release_to_pool(Block* blk) {
    DeviceState& st = state(blk->device);
    if (blk->pool != 0 && retired_pools_.count(blk->pool)) blk->pool = 0;  // its graph is gone: back to the shared cache
    Pool& pool = blk->small ? st.small_free : st.large_free;
    // Merge with free neighbours of the same segment.
    auto absorb = [&](Block* nb, bool nb_is_prev) {
      if (!nb || nb->in_use || nb->pending_events > 0) return;
      auto it = pool.find(nb);
      if (it == pool.end()) return;  // still waiting on notifiers
      pool.erase(it);
      if (nb_is_prev) {
        blk->ptr = nb->ptr;
        blk->prev = nb->prev;
        if (blk->prev) blk->prev->next = blk;
      } else {
        blk->next = nb->next;
        if (blk->next) blk->next->prev = blk;
      }
      blk->size += nb->size;
      delete nb;
    };
    absorb(blk->prev, true);
    absorb(blk->next, false);
    pool.insert(blk);
  }

  void drain_pending(DeviceState& st) {
    while (!st.pending.empty()) {
      PendingFree& pf = st.pending.front();
      if (!pf.n->query()) break;
      finish_pending(pf);
      st.pending.pop_front();
    }
  }
  void sync_pending(DeviceState& st) {
    while (!st.pending.empty()) {
      PendingFree& pf = st.pending.front();
      pf.n->synchronize();
      finish_pending(pf);
      st.pending.pop_front();
    }
  }
  void finish_pending(PendingFree& pf) {
    NotifierPool::instance().give_back(std::move(pf.n), pf.block->device);
    if (--pf.block->pending_events == 0) release_to_pool(pf.block);
  }

  void release_segments(DeviceState& st, Pool& pool, int device) {
    DeviceSwitch sw(device);
    for (auto it = pool.begin(); it != pool.end();) {
      Block* b = *it;
      if (b->prev == nullptr && b->next == nullptr && b->pool == 0) {  // a whole segment is free (graph pools keep theirs)
        backend().free(b->ptr);
        st.stats.reserved -= static_cast<int64_t>(b->size);
        st.stats.num_segments--;
        it = pool.erase(it);
        delete b;
      } else {
        ++it;
      }
    }
  }

  // ------------------------------------------------------------- debug mode
  void record_origin(Block* b, std::string context) {
    void* frames[24];
    const int n = ::backtrace(frames, 24);
    b->origin_frames.assign(frames + std::min(n, 2), frames + n);  // without this function and malloc_block()
    b->origin_context = std::move(context);
  }
  static std::string format_origin(const Block* b) {
    if (b->origin_frames.empty() && b->origin_context.empty()) return "";
    std::ostringstream os;
    os << "  allocated at:\n";
    if (!b->origin_context.empty()) os << b->origin_context;
    char** names = ::backtrace_symbols(b->origin_frames.data(), static_cast<int>(b->origin_frames.size()));
    for (size_t i = 0; names && i < b->origin_frames.size(); ++i) {
      // "module(mangled+0x12) [addr]" -> demangle the part between '(' and '+'
      std::string line = names[i];
      const size_t l = line.find('('), r = line.find('+', l == std::string::npos ? 0 : l);
      if (l != std::string::npos && r != std::string::npos && r > l + 1) {
        line = line.substr(0, l + 1) + c10::demangle(line.substr(l + 1, r - l - 1).c_str()) + line.substr(r);
      }
      os << "    " << line << "\n";
    }
    std::free(names);
    return os.str();
  }
  void paint_guards(Block* b, const Queue& q) {
    DeviceSwitch sw(b->device);
    backend().memset_async(b->ptr, kGuardByte, kGuard, q.handle());
    backend().memset_async(b->ptr + b->size - kGuard, kGuardByte, kGuard, q.handle());
  }
  bool verify_guards(Block* b, std::string* why) {
    std::array<uint8_t, 2 * kGuard> host;
    DeviceSwitch sw(b->device);
    synchronize(b->device);
    void* s = getDefaultQueue(b->device).handle();
    backend().memcpy_async(host.data(), b->ptr, kGuard, CopyKind::D2H, s);
    backend().memcpy_async(host.data() + kGuard, b->ptr + b->size - kGuard, kGuard, CopyKind::D2H, s);
    backend().stream_synchronize(s);
    int head_bad = -1, tail_bad = -1;
    for (size_t i = 0; i < kGuard; ++i) {
      if (host[i] != kGuardByte) head_bad = static_cast<int>(i);  // last damaged byte before the block
    }
    for (size_t i = 0; i < kGuard; ++i) {
      if (host[kGuard + i] != kGuardByte) {
        tail_bad = static_cast<int>(i);  // first damaged byte after the block
        break;
      }
    }
    if (head_bad < 0 && tail_bad < 0) return true;
    std::ostringstream os;
    os << "block " << static_cast<void*>(b->ptr + kGuard) << " (" << b->requested << " B requested, device "
       << b->device << ")";
    if (head_bad >= 0) os << " header guard damaged " << (kGuard - head_bad) << " B before the block";
    if (tail_bad >= 0) os << " footer guard damaged " << tail_bad << " B after the rounded block end";
    const std::string origin = format_origin(b);
    if (!origin.empty()) os << "\n" << origin;
    *why = os.str();
    return false;
  }

  std::recursive_mutex mu_;
  std::array<std::unique_ptr<DeviceState>, kMaxDevices> states_;
  std::unordered_map<void*, Block*> live_;
  uint64_t next_pool_ = 0;
  std::unordered_set<uint64_t> retired_pools_;
  bool native_ = false;
  bool debug_ = false;
  int64_t corrupted_on_free_ = 0;
  std::string last_corruption_;
};

CachingAllocator& alloc() {
  static CachingAllocator* a = new CachingAllocator();  // leaked on purpose
  return *a;
}

void CachingAllocator::deleter(void* p) {
  try {
    alloc().free_block(p);
  } catch (const std::exception& e) {
    B200LOG(ERROR) << "b200 allocator: exception while freeing: " << e.what();
  }
}

}  // namespace

c10::Allocator* getB200CachingAllocator() { return &alloc(); }
void* raw_alloc(size_t bytes, int device, const Queue& q) { return alloc().malloc_block(bytes, device, q); }
void raw_free(void* ptr) { alloc().free_block(ptr); }
void recordQueue(const c10::DataPtr& ptr, const Queue& q) { alloc().record_queue(ptr.get(), q); }
void recordQueueRaw(void* ptr, const Queue& q) { alloc().record_queue(ptr, q); }
namespace {
std::mutex g_dropper_mu;
std::vector<std::function<void()>> g_droppers;
}  // namespace
void registerCacheDropper(std::function<void()> fn) {
  std::lock_guard<std::mutex> lk(g_dropper_mu);
  g_droppers.push_back(std::move(fn));
}
void emptyCache() {
  std::vector<std::function<void()>> fns;
  {
    std::lock_guard<std::mutex> lk(g_dropper_mu);
    fns = g_droppers;
  }
  for (auto& f : fns) f();  // upper layers release the device tensors their own caches keep alive
  alloc().empty_cache();
}
MemoryStats memoryStats(int device) { return alloc().stats(device); }
void resetPeakStats(int device) { alloc().reset_peak(device); }
void setNativeMemoryStrategy(bool native) { alloc().set_native(native); }
bool nativeMemoryStrategy() { return alloc().native(); }
void setMemoryFraction(double fraction, int device) {
  TORCH_CHECK(fraction >= 0.0 && fraction <= 1.0, "invalid memory fraction ", fraction, " (expected a value in [0, 1]; 0 lifts the limit)");
  int64_t limit = 0;
  if (fraction > 0.0) {
    DeviceSwitch sw(device);
    size_t free_b = 0, total_b = 0;
    backend().mem_info(&free_b, &total_b);
    limit = static_cast<int64_t>(fraction * static_cast<double>(total_b));
  }
  alloc().set_reserve_limit(device, limit);
}
int64_t memoryReserveLimit(int device) { return alloc().reserve_limit(device); }
void setMemoryDebug(bool on) { alloc().set_debug(on); }
bool memoryDebugEnabled() { return alloc().debug(); }
DebugReport memoryDebugCheck(const void* ptr) { return alloc().debug_check(ptr); }
uint64_t newPrivatePool() { return alloc().new_pool(); }
uint64_t setThreadPrivatePool(uint64_t pool) {
  const uint64_t prev = t_private_pool;
  t_private_pool = pool;
  return prev;
}
void retirePrivatePool(uint64_t pool) { alloc().retire_pool(pool); }
void setAllocationContextHook(AllocationContextHook hook) { g_context_hook.store(hook); }
std::string memoryDebugOrigin(const void* ptr) { return alloc().origin_of(ptr); }
std::string memorySummary(int device) { return alloc().summary(device); }

}  // namespace catch_b200
