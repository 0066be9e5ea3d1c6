// Per-device, queue-aware caching allocator for device memory.
//
// Capability parity with torch_mlu/csrc/aten/core/caching_allocator.cpp
// (constants :58-69, stats :97-124, malloc/free :330-425, recordQueue :578-599,
// debug allocator :612-762, public API :805-886):
//   * 512-byte rounding, requests <= 1 MiB are carved from 2 MiB segments,
//     bigger ones from segments of at least 20 MiB (or exact 2 MiB multiples)
//   * best-fit lookup per (queue, size), split on allocation, merge on free
//   * a block used on other queues (recordQueue) is returned to the pool only
//     after notifiers placed on those queues have been reached
//   * out-of-memory: release all cached segments and retry once, then raise
//     an error that lists the totals
//   * statistics: allocated / max_allocated / reserved(cached) / max_reserved
//   * optional debug mode: guard regions before and after each block that are
//     verified when the block is freed and on demand
// The data structures are this project's own (intrusive doubly linked segment
// lists plus two ordered sets per device).
#pragma once
#include <functional>
#include <c10/core/Allocator.h>
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>
#include "queue.h"

namespace catch_b200 {

struct MemoryStats {
  int64_t allocated = 0;
  int64_t max_allocated = 0;
  int64_t reserved = 0;
  int64_t max_reserved = 0;
  int64_t num_alloc = 0;
  int64_t num_free = 0;
  int64_t num_segments = 0;
  int64_t num_ooms = 0;
  int64_t num_retries = 0;
};

struct DebugReport {
  int64_t blocks_checked = 0;
  int64_t corrupted = 0;
  std::string detail;  // one line per corrupted block
};

c10::Allocator* getB200CachingAllocator();

// Raw interface used by operators for workspaces.
void* raw_alloc(size_t bytes, int device, const Queue& q);
void raw_free(void* ptr);

void recordQueue(const c10::DataPtr& ptr, const Queue& q);
void recordQueueRaw(void* ptr, const Queue& q);
void emptyCache();
// Layers above the runtime that cache device tensors (quantized weights, scale copies) register a
// function that drops them; emptyCache() runs these first so that the memory really returns.
void registerCacheDropper(std::function<void()> fn);
MemoryStats memoryStats(int device);
void resetPeakStats(int device);
// true = allocate exactly what is asked from the driver (no over-sized
// segments); false (default) = cache-friendly segment sizes.
void setNativeMemoryStrategy(bool native);
bool nativeMemoryStrategy();
// Cap on the device memory this process's allocator may hold, as a fraction of the device's capacity (0 = no cap;
// torch.cuda.set_per_process_memory_fraction semantics: a request that would exceed it fails like an out-of-memory
// condition, after cached blocks were given back).
void setMemoryFraction(double fraction, int device);
int64_t memoryReserveLimit(int device);
// Debug allocator: enable before the first allocation (or via the environment).
void setMemoryDebug(bool on);
bool memoryDebugEnabled();
DebugReport memoryDebugCheck(const void* ptr = nullptr);  // nullptr = every live block
// In memory-debug mode every block remembers where it was allocated (reference: the debug allocator's recorded
// backtraces, torch_mlu/csrc/aten/core/caching_allocator.cpp:633): the native return addresses, symbolised only when a
// report is written, plus the text this hook returns at allocation time (the binding layer installs one that walks
// the Python frames of the calling thread).
// Private pools for captured graphs: while a thread has a pool set, its allocations come from (and its frees of
// such blocks return to) segments that only this pool uses; retirePrivatePool hands them to the shared cache.
uint64_t newPrivatePool();
uint64_t setThreadPrivatePool(uint64_t pool);  // returns the previous value; 0 = shared cache
void retirePrivatePool(uint64_t pool);

using AllocationContextHook = std::string (*)();
void setAllocationContextHook(AllocationContextHook hook);
std::string memoryDebugOrigin(const void* ptr);  // "" when the block has no record
std::string memorySummary(int device);

}  // namespace catch_b200
