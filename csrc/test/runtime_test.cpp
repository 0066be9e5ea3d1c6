// Self-checking C++ tests of the native runtime: device, queues and the queue pool,
// notifiers, the caching allocator (reuse, splitting, statistics, cross-queue deferral,
// debug guards), the pinned host allocator, the device guard and tensor construction.
// Runs against whichever backend is selected (host simulation without a GPU).
//
// Mirrors the reference's gtest suite (torch_mlu/csrc/test/aten/{caching_allocator_test,
// queue_test,queue_pool_test,notifier_test,guard_test,memory_allocator_test,
// tensor_util_test}.cpp) without depending on gtest: every CHECK_T failure is counted and
// the process exits non-zero if any occurred.
#include <ATen/ATen.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>

#include <cstdio>
#include <cstring>
#include <set>
#include <string>
#include <thread>
#include <vector>

#include "../runtime/backend.h"
#include "../runtime/caching_allocator.h"
#include "../runtime/device.h"
#include "../runtime/host_allocator.h"
#include "../runtime/notifier.h"
#include "../runtime/queue.h"
#include "../runtime/tensor_impl.h"

using namespace catch_b200;

int g_failures = 0, g_checks = 0;  // shared with jit_test.cpp
#define CHECK_T(cond)                                                              \
  do {                                                                             \
    ++g_checks;                                                                    \
    if (!(cond)) {                                                                 \
      ++g_failures;                                                                \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);       \
    }                                                                              \
  } while (0)

static void test_device() {
  CHECK_T(device_count() >= 1);
  set_device(0);
  CHECK_T(current_device() == 0);
  const DeviceProp& p = device_properties(0);
  CHECK_T(!p.name.empty());
  CHECK_T(p.total_memory > 0);
  {
    DeviceSwitch sw(device_count() - 1);
    CHECK_T(current_device() == device_count() - 1);
  }
  CHECK_T(current_device() == 0);
  CHECK_T(!version_string().empty());
  synchronize();
}

static void test_queues() {
  Queue d = getDefaultQueue(0);
  CHECK_T(d.is_default() && d.id() == 0 && d.device_index() == 0);
  CHECK_T(getCurrentQueue(0) == d);
  // the pool hands out its 32 queues round robin
  std::set<int> ids;
  Queue first = getQueueFromPool(0);
  ids.insert(first.id());
  for (int i = 1; i < 32; ++i) ids.insert(getQueueFromPool(0).id());
  CHECK_T(ids.size() == 32);
  CHECK_T(getQueueFromPool(0) == first);
  CHECK_T(!first.is_default());
  CHECK_T(getQueueById(0, first.id()) == first);
  // current queue is per thread
  {
    QueueGuard g(first);
    CHECK_T(getCurrentQueue(0) == first);
    std::thread t([&] { CHECK_T(getCurrentQueue(0) == getDefaultQueue(0)); });
    t.join();
  }
  CHECK_T(getCurrentQueue(0) == d);
  setCurrentQueue(first);
  CHECK_T(getCurrentQueue(0) == first);
  setCurrentQueue(d);
  CHECK_T(first.query());
  first.synchronize();
  CHECK_T(Queue::from_c10(first.to_c10()) == first);
  CHECK_T(std::hash<Queue>()(first) != std::hash<Queue>()(d));
  synchronizeAllQueues(0);
}

static void test_notifiers() {
  Notifier never;
  CHECK_T(never.query());  // never placed counts as reached
  Queue q = getQueueFromPool(0);
  Notifier a(true), b(true);
  a.place(q);
  b.place(q);
  b.synchronize();
  CHECK_T(a.query() && b.query());
  CHECK_T(a.elapsed_time(b) >= 0.f);
  CHECK_T(a.hardware_time(b) >= 0.f);
  // another queue waits for the marker
  Queue q2 = getQueueFromPool(0);
  a.wait(q2);
  q2.synchronize();
  Notifier moved(std::move(b));
  CHECK_T(moved.query());
  NotifierPool& pool = NotifierPool::instance();
  pool.clean();
  auto n = pool.alloc(0);
  n->place(q);
  n->synchronize();
  pool.give_back(std::move(n), 0);
  CHECK_T(pool.cached(0) == 1);
  auto again = pool.alloc(0);
  CHECK_T(pool.cached(0) == 0);
}

static void test_caching_allocator() {
  emptyCache();
  resetPeakStats(0);
  const MemoryStats s0 = memoryStats(0);
  Queue q = getCurrentQueue(0);
  void* a = raw_alloc(1000, 0, q);
  CHECK_T(a != nullptr);
  MemoryStats s1 = memoryStats(0);
  CHECK_T(s1.allocated - s0.allocated == 1024);  // rounded up to 512-byte multiples
  CHECK_T(s1.reserved >= s0.reserved + (2 << 20));  // small requests are carved from 2 MiB segments
  void* b = raw_alloc(3000, 0, q);
  CHECK_T(static_cast<char*>(b) == static_cast<char*>(a) + 1024);  // split of the same segment
  raw_free(a);
  void* c = raw_alloc(512, 0, q);
  CHECK_T(c == a);  // best fit reuses the freed block
  raw_free(b);
  raw_free(c);
  MemoryStats s2 = memoryStats(0);
  CHECK_T(s2.allocated == s0.allocated);
  CHECK_T(s2.max_allocated >= s1.allocated);
  CHECK_T(s2.num_alloc - s0.num_alloc == 3 && s2.num_free - s0.num_free == 3);
  // a large block gets its own segment
  void* big = raw_alloc(32 << 20, 0, q);
  CHECK_T(memoryStats(0).reserved >= s2.reserved + (32 << 20));
  raw_free(big);
  emptyCache();
  CHECK_T(memoryStats(0).reserved == 0 || memoryStats(0).reserved <= s0.reserved);
  // a block used on another queue is not handed out again before that queue has passed the free
  Queue other = getQueueFromPool(0);
  void* x = raw_alloc(4096, 0, q);
  recordQueueRaw(x, other);
  raw_free(x);
  other.synchronize();
  void* y = raw_alloc(4096, 0, q);
  CHECK_T(y != nullptr);
  raw_free(y);
  CHECK_T(!memorySummary(0).empty());
  // c10 allocator interface
  c10::DataPtr dp = getB200CachingAllocator()->allocate(100);
  CHECK_T(dp.get() != nullptr && dp.device().type() == c10::DeviceType::PrivateUse1);
}

static void test_debug_allocator() {
  emptyCache();
  setMemoryDebug(true);
  CHECK_T(memoryDebugEnabled());
  Queue q = getCurrentQueue(0);
  void* p = raw_alloc(256, 0, q);
  CHECK_T(memoryDebugCheck(p).corrupted == 0);
  CHECK_T(memoryDebugCheck().blocks_checked >= 1);
  if (backend().is_hostsim()) {
    // device memory is host memory here: write one byte past the (512-byte rounded) block and expect
    // the footer guard to notice
    static_cast<unsigned char*>(p)[512] ^= 0xff;
    DebugReport r = memoryDebugCheck(p);
    CHECK_T(r.corrupted == 1 && !r.detail.empty());
    static_cast<unsigned char*>(p)[512] ^= 0xff;
    CHECK_T(memoryDebugCheck(p).corrupted == 0);
  }
  raw_free(p);
  setMemoryDebug(false);
  emptyCache();
}

static void test_native_strategy() {
  emptyCache();
  setNativeMemoryStrategy(true);
  CHECK_T(nativeMemoryStrategy());
  Queue q = getCurrentQueue(0);
  void* p = raw_alloc(1 << 20, 0, q);
  CHECK_T(p != nullptr);
  raw_free(p);
  setNativeMemoryStrategy(false);
  CHECK_T(!nativeMemoryStrategy());
}

static void test_pinned_allocator() {
  pinnedEmptyCache();
  c10::Allocator* pa = getB200PinnedAllocator();
  void* first;
  {
    c10::DataPtr h = pa->allocate(1 << 16);
    first = h.get();
    CHECK_T(first != nullptr && isPinnedPtr(first));
    CHECK_T(isPinnedPtr(static_cast<char*>(first) + 100));
    std::memset(first, 7, 1 << 16);
  }
  CHECK_T(pinnedCachedBytes() >= (1 << 16));
  {
    c10::DataPtr h = pa->allocate(1 << 16);
    CHECK_T(h.get() == first);  // served from the cache
  }
  int on_stack = 0;
  CHECK_T(!isPinnedPtr(&on_stack));
  pinnedEmptyCache();
  CHECK_T(pinnedCachedBytes() == 0);
}

static void test_guard() {
  const c10::impl::DeviceGuardImplInterface* impl = c10::impl::getDeviceGuardImpl(c10::DeviceType::PrivateUse1);
  CHECK_T(impl != nullptr && impl->type() == c10::DeviceType::PrivateUse1);
  CHECK_T(impl->deviceCount() == device_count());
  const c10::Device d0(c10::DeviceType::PrivateUse1, 0);
  impl->setDevice(d0);
  CHECK_T(impl->getDevice() == d0);
  const c10::Device last(c10::DeviceType::PrivateUse1, (c10::DeviceIndex)(device_count() - 1));
  const c10::Device prev = impl->exchangeDevice(last);
  CHECK_T(prev == d0 && impl->getDevice() == last);
  impl->uncheckedSetDevice(d0);
  // streams: exchanging installs the new current queue and returns the old one
  Queue q = getQueueFromPool(0);
  const c10::Stream old = impl->exchangeStream(q.to_c10());
  CHECK_T(Queue::from_c10(old) == getDefaultQueue(0));
  CHECK_T(Queue::from_c10(impl->getStream(d0)) == q);
  impl->exchangeStream(old);
  CHECK_T(getCurrentQueue(0) == getDefaultQueue(0));
}

static void test_tensors() {
  at::Tensor t = empty_b200({4, 5}, at::kFloat, 0);
  CHECK_T(is_b200(t) && t.numel() == 20 && t.is_contiguous());
  CHECK_T(maybe_b200_impl(t) != nullptr);
  at::Tensor cl = empty_b200({2, 8, 3, 3}, at::kHalf, 0, at::MemoryFormat::ChannelsLast);
  CHECK_T(cl.is_contiguous(at::MemoryFormat::ChannelsLast) && cl.stride(1) == 1);
  at::Tensor st = empty_strided_b200({3, 4}, {1, 3}, at::kLong, 0);
  CHECK_T(st.stride(0) == 1 && st.stride(1) == 3);
  // host -> device -> host through the backend's copy primitive (the ATen copy kernels live in the
  // operator library, which this program does not link)
  at::Tensor cpu = at::arange(20, at::kFloat).view({4, 5});
  at::Tensor back = at::zeros({4, 5}, at::kFloat);
  Queue q = getCurrentQueue(0);
  backend().memcpy_async(t.data_ptr(), cpu.data_ptr(), 20 * sizeof(float), CopyKind::H2D, q.handle());
  backend().memcpy_async(back.data_ptr(), t.data_ptr(), 20 * sizeof(float), CopyKind::D2H, q.handle());
  q.synchronize();
  CHECK_T(at::equal(back, cpu));
  CHECK_T(!is_b200(cpu) && !is_b200(at::Tensor()));
}

void test_jit_lowering();
void test_jit_partitioner();
void test_jit_alias_safety();
void test_jit_runner_cache();
void test_check_util();

int main() {
  struct Case { const char* name; void (*fn)(); };
  const Case cases[] = {{"device", test_device},           {"queues", test_queues},
                        {"notifiers", test_notifiers},     {"caching_allocator", test_caching_allocator},
                        {"debug_allocator", test_debug_allocator}, {"native_strategy", test_native_strategy},
                        {"pinned_allocator", test_pinned_allocator}, {"guard", test_guard},
                        {"tensors", test_tensors},         {"check_util", test_check_util},
                        {"jit_lowering", test_jit_lowering}, {"jit_partitioner", test_jit_partitioner},
                        {"jit_alias_safety", test_jit_alias_safety}, {"jit_runner_cache", test_jit_runner_cache}};
  for (const Case& c : cases) {
    const int before = g_failures;
    try {
      c.fn();
    } catch (const std::exception& e) {
      ++g_failures;
      std::fprintf(stderr, "FAILED %s: exception: %s\n", c.name, e.what());
    }
    std::printf("[%s] %s\n", g_failures == before ? "  OK  " : "FAILED", c.name);
  }
  std::printf("%d checks, %d failures\n", g_checks, g_failures);
  if (g_failures == 0) std::printf("ALL PASSED\n");
  return g_failures == 0 ? 0 : 1;
}
